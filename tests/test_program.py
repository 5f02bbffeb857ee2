"""Expressions outside the seven score functions: compiled to a register program (cuke_b200.program) and run by the
general evaluator (kge_eval_program).  Golden outputs come from the reference's own generator and C++ back-end for the
same expressions (tests/golden/make_program_golden.py -> tests/golden/program.npz)."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import program_model

Z = np.load(os.path.join(os.path.dirname(__file__), "golden", "program.npz"))
NAMES = ["plain_dot", "scaled_mix", "project_product", "outer_of_difference", "scaled_outer", "scaled_rows", "two_hop"]


def build(name):
    """The expressions of tests/golden/make_program_golden.py, written against cuke_b200's surface."""
    from cuke_b200 import kge
    from cuke_b200.asg import Tensor, Var
    bvv, bsv, bvm, bov, bsm = kge.bvv, kge.bsv, kge.bvm, kge.bov, kge.bsm
    nnodes, nedges, dim, batch = Var(name="nnodes"), Var(name="nedges"), Var(name="dim"), Var(name="batch_size")
    h = Tensor((batch,), dtype="int", name="h"); t = Tensor((batch,), dtype="int", name="t"); r = Tensor((batch,), dtype="int", name="r")
    E = Tensor((nnodes, dim), name="Eemb"); R = Tensor((nedges, dim), name="Remb"); M = Tensor((nedges, dim, dim), name="Proj")
    dout = Tensor((batch,), name="dout")
    return {"plain_dot": lambda: bvv(E[h], E[t]),
            "scaled_mix": lambda: bsv(bvv(E[h], R[r]), E[t]) - E[h] * R[r],
            "project_product": lambda: bvm(E[h] * R[r], M[r]) + E[t],
            "outer_of_difference": lambda: bov(E[h] - E[t], R[r]),
            "scaled_outer": lambda: bsm(dout, bov(E[h], E[t])),
            "scaled_rows": lambda: bsv(dout, E[h] - E[t] + R[r]),
            "two_hop": lambda: bvv(bvm(bvm(E[h], M[r]), M[r]), E[t])}[name]()


def rel_err(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max() / max(np.abs(b).max(), 1e-30))


@pytest.mark.parametrize("name", NAMES)
def test_compiled_program_matches_reference_output(name):
    """CPU: positional order as the reference's generated function takes it, and the program's semantics (numpy
    interpreter) against the reference's output."""
    from cuke_b200.codegen import gpu
    desc = json.loads(gpu.print_cuda(build(name)))
    assert desc["model"] == "program"
    assert desc["args"] == Z["args_" + name].tolist()
    prog = desc["program"]
    tables = [Z[n] for n in prog["tables"]]
    ids = [Z[n].astype(np.int64) for n in prog["ids"]]
    out = program_model.run(prog, tables, ids, int(Z["h"].shape[0]), int(Z["Eemb"].shape[1]))
    ref = Z["out_" + name]
    assert out.shape == ref.shape
    assert rel_err(out, ref) < 1e-5


def test_score_functions_still_take_their_own_kernels():
    from cuke_b200 import kge
    from cuke_b200.codegen import gpu
    assert json.loads(kge.transE())["model"] == "TransE"
    assert json.loads(kge.RESCAL())["model"] == "RESCAL"


def test_unsupported_expressions_say_so():
    from cuke_b200.asg import Tensor, Var
    from cuke_b200.codegen import gpu
    b, d = Var(name="batch_size"), Var(name="dim")
    h = Tensor((b,), dtype="int", name="h")
    with pytest.raises(NotImplementedError):
        gpu.print_cuda(h + h)                       # an index tensor is not a value


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_general_evaluator_on_gpu(name, idt):
    from cuke_b200 import run
    from cuke_b200.codegen import gpu
    code = gpu.print_cuda(build(name))
    scal = {"batch_size": int(Z["h"].shape[0]), "dim": int(Z["Eemb"].shape[1]), "nnodes": int(Z["Eemb"].shape[0]), "nedges": int(Z["Remb"].shape[0])}
    args = []
    for a in Z["args_" + name].tolist():
        if a in scal:
            args.append(scal[a])
        elif a in ("h", "r", "t"):
            args.append(torch.from_numpy(Z[a].astype(np.int64)).to(idt).cuda())
        else:
            args.append(torch.from_numpy(Z[a]).cuda())
    out = run.gpu.compile_and_run(code, *args)
    ref = Z["out_" + name]
    assert tuple(out.shape) == ref.shape
    assert rel_err(out.cpu().numpy(), ref) < 1e-5
    assert torch.equal(out, run.gpu.compile_and_run(code, *args))


@pytest.mark.gpu
def test_general_evaluator_at_embedding_size():
    """dim 400 (the largest benchmark dim), batch not a multiple of the warps per block."""
    from cuke_b200 import run
    from cuke_b200.codegen import gpu
    g = np.random.default_rng(4)
    ne, nr, d, B = 300, 7, 400, 1001
    E = (g.standard_normal((ne, d)) / 20).astype(np.float32); R = (g.standard_normal((nr, d)) / 20).astype(np.float32)
    h, r, t = g.integers(0, ne, B), g.integers(0, nr, B), g.integers(0, ne, B)
    code = gpu.print_cuda(build("scaled_mix"))
    dev = lambda a: torch.from_numpy(a).cuda()
    out = run.gpu.compile_and_run(code, B, d, ne, dev(E), dev(h), nr, dev(R), dev(r), dev(t))
    ref = (E[h] * R[r]).sum(1, keepdims=True) * E[t] - E[h] * R[r]
    assert rel_err(out.cpu().numpy(), ref) < 1e-5
