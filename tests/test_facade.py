"""Host-side logic that needs no GPU: the pycuke1-style front-end, recognition of the score functions, the
positional argument order, and the C-ABI library's exported symbols."""
import ctypes
import json
import os
import re

import pytest

from cuke_b200 import kge, transform
from cuke_b200.asg import Tensor, Var
from cuke_b200.asg2ir import gen_ir
from cuke_b200.codegen import gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# positional run(...) lists of the reference's generated wrappers (pycuke1/helpers.py:179-190 applied to
# apps/kge/kge.py:273-390; call sites apps/kge/test_cuke.py:54,104,153,198,244)
REFERENCE_ARGS = {
    "transE": "batch_size, dim, nnodes, Eemb, h, t, nedges, Remb, r, r_uniq, r_buf, r_unique_cnt",
    "transH": "batch_size, dim, nnodes, Eemb, h, t, nedges, Remb, r, r_uniq, r_buf, r_unique_cnt, Pemb",
    "transR": "batch_size, dim, nnodes, Eemb, h, t, nedges, Proj, r, r_uniq, r_buf, r_unique_cnt, Remb",
    "transF": "batch_size, dim, nnodes, Eemb, h, nedges, Remb, r, r_uniq, r_buf, r_unique_cnt, t",
    "RESCAL": "batch_size, dim, nnodes, Eemb, h, nedges, Proj, r, r_uniq, r_buf, r_unique_cnt, t",
}
MODEL_OF = {"transE": "TransE", "transH": "TransH", "transR": "TransR", "transF": "TransF", "RESCAL": "RESCAL",
            "distmult": "DistMult", "complEx": "ComplEx"}


@pytest.mark.parametrize("fn", list(MODEL_OF))
def test_entry_points_recognised(fn):
    d = json.loads(getattr(kge, fn)())
    assert d["model"] == MODEL_OF[fn]
    if fn in REFERENCE_ARGS:
        assert ", ".join(d["args"]) == REFERENCE_ARGS[fn]


def _base():
    nnodes, nedges, dim, batch = Var(name='nnodes'), Var(name='nedges'), Var(name='dim'), Var(name='batch_size')
    h = Tensor((batch,), dtype='int', name='heads'); t = Tensor((batch,), dtype='int', name='tails')
    r = Tensor((batch,), dtype='int', name='rels')
    return nnodes, nedges, dim, batch, h, t, r


def test_no_reuse_means_no_side_tables():
    # apps/kge/test_cuke.py:27-54: TransE without r.attr['reuse'] takes nine arguments
    nnodes, nedges, dim, batch, h, t, r = _base()
    E = Tensor((nnodes, dim), name='ent'); R = Tensor((nedges, dim), name='relv')
    d = json.loads(gpu.print_cuda(gen_ir(E[h] - E[t] + R[r])))
    assert d["model"] == "TransE"
    assert d["args"] == ["batch_size", "dim", "nnodes", "ent", "heads", "tails", "nedges", "relv", "rels"]
    assert d["roles"]["Eemb"] == "ent" and d["roles"]["h"] == "heads" and d["roles"]["r"] == "rels"


def test_recognition_is_structural():
    nnodes, nedges, dim, batch, h, t, r = _base()
    E = Tensor((nnodes, dim), name='ent'); R = Tensor((nedges, dim), name='relv'); W = Tensor((nedges, dim), name='nrm')
    # TransE written in another order; TransH with the dot product's operands swapped
    assert json.loads(gpu.print_cuda(gen_ir(R[r] + E[h] - E[t])))["model"] == "TransE"
    u = E[h] - E[t]
    d = json.loads(gpu.print_cuda(gen_ir(u + R[r] - kge.bsv(kge.bvv(u, W[r]), W[r]))))
    assert d["model"] == "TransH" and d["roles"]["Pemb"] == "nrm" and d["roles"]["Remb"] == "relv"
    # head and tail exchanged is NOT TransE's h - t + r with the same roles: roles follow the expression
    d = json.loads(gpu.print_cuda(gen_ir(E[t] - E[h] + R[r])))
    assert d["model"] == "TransE" and d["roles"]["h"] == "tails" and d["roles"]["t"] == "heads"
    # expressions that are none of the seven score functions are compiled for the general evaluator instead
    assert json.loads(gpu.print_cuda(gen_ir(E[h] + E[t] + R[r])))["model"] == "program"
    assert json.loads(gpu.print_cuda(gen_ir(kge.bvv(E[h], E[t]))))["model"] == "program"


def test_passes_list_is_the_reference_default():
    assert [type(p).__name__ for p in transform.passes] == ["fuser", "tiler", "smem", "indirect_smem"]


def test_cpu_paths_refuse():
    from cuke_b200 import codegen, run
    with pytest.raises(NotImplementedError):
        codegen.cpu.print_cpp(None)
    with pytest.raises(NotImplementedError):
        run.cpu.compile_and_run("")


def test_library_exports_every_declared_symbol():
    from cuke_b200 import _lib
    header = open(os.path.join(ROOT, "include", "kge_b200.h")).read()
    declared = set(re.findall(r"KGE_API\s+[\w\s\*]+?\b(kge_\w+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.SIGNATURES), "ctypes table and header disagree"
    if not os.path.exists(_lib.LIB_PATH):
        pytest.skip("library not built")
    L = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(L, name), f"{name} not exported"
    assert _lib.lib().kge_version() == 1


def test_install_as_pycuke1():
    import sys
    import cuke_b200
    cuke_b200.install_as_pycuke1()
    import pycuke1
    from pycuke1.asg import Tensor as T2
    from pycuke1 import run as run2
    assert T2 is Tensor and hasattr(run2.gpu, "compile_and_run")
    for k in [k for k in sys.modules if k == "pycuke1" or k.startswith("pycuke1.") or k == "kge"]:
        del sys.modules[k]
