"""Golden outputs for expressions OUTSIDE the seven score functions, produced by the reference's own generator.

    CUKE_REFERENCE=<cuke checkout> python tests/golden/make_program_golden.py

Each expression is written with the reference's operators (apps/kge/kge.py:13-35: bvv, bsv, bvm, bov, bsm), lowered with
pycuke1.asg2ir.gen_ir, printed with pycuke1.codegen.cpu.print_cpp (passes = [kge.fuser()], the CPU-compilable pipeline),
compiled with torch.utils.cpp_extension and run on seeded inputs; inputs and outputs go to tests/golden/program.npz.
The positional argument order is read from the generated function's own signature.  The same expressions are written
against cuke_b200's surface in tests/test_program.py (EXPRESSIONS must stay in step with it)."""
import os
import re
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
NE, NR, D, B = 41, 6, 20, 33


def expressions(ns):
    """name -> root node, over tensors Eemb (nnodes, dim), Remb (nedges, dim), Proj (nedges, dim, dim), dout (batch,),
    h, r, t (batch,) int."""
    Var, Tensor = ns["Var"], ns["Tensor"]
    bvv, bsv, bvm, bov, bsm = ns["bvv"], ns["bsv"], ns["bvm"], ns["bov"], ns["bsm"]

    def leaves():
        nnodes, nedges, dim, batch = Var(name="nnodes"), Var(name="nedges"), Var(name="dim"), Var(name="batch_size")
        h = Tensor((batch,), dtype="int", name="h"); t = Tensor((batch,), dtype="int", name="t"); r = Tensor((batch,), dtype="int", name="r")
        E = Tensor((nnodes, dim), name="Eemb"); R = Tensor((nedges, dim), name="Remb"); M = Tensor((nedges, dim, dim), name="Proj")
        dout = Tensor((batch,), name="dout")
        return h, t, r, E, R, M, dout
    out = {}
    h, t, r, E, R, M, dout = leaves(); out["plain_dot"] = bvv(E[h], E[t])
    h, t, r, E, R, M, dout = leaves(); out["scaled_mix"] = bsv(bvv(E[h], R[r]), E[t]) - E[h] * R[r]
    h, t, r, E, R, M, dout = leaves(); out["project_product"] = bvm(E[h] * R[r], M[r]) + E[t]
    h, t, r, E, R, M, dout = leaves(); out["outer_of_difference"] = bov(E[h] - E[t], R[r])
    h, t, r, E, R, M, dout = leaves(); out["scaled_outer"] = bsm(dout, bov(E[h], E[t]))          # apps/kge/kge.py:450-451 pattern
    h, t, r, E, R, M, dout = leaves(); out["scaled_rows"] = bsv(dout, E[h] - E[t] + R[r])
    h, t, r, E, R, M, dout = leaves(); out["two_hop"] = bvv(bvm(bvm(E[h], M[r]), M[r]), E[t])
    return out


def main():
    ref = os.environ.get("CUKE_REFERENCE", os.path.join(HERE, "..", "..", "..", "reference"))
    sys.path[:0] = [ref, os.path.join(ref, "apps", "kge")]
    sys.dont_write_bytecode = True
    os.environ["CXX"], os.environ["CC"] = "/usr/bin/g++", "/usr/bin/gcc"
    import torch
    import kge  # the reference's apps/kge/kge.py
    from pycuke1 import transform
    from pycuke1.asg import Tensor, Var
    from pycuke1.asg2ir import gen_ir
    from pycuke1.codegen import cpu
    from torch.utils.cpp_extension import load
    ns = dict(Var=Var, Tensor=Tensor, bvv=kge.bvv, bsv=kge.bsv, bvm=kge.bvm, bov=kge.bov, bsm=kge.bsm)
    g = np.random.Generator(np.random.PCG64(777))
    data = {"Eemb": (g.standard_normal((NE, D)) / np.sqrt(D)).astype(np.float32),
            "Remb": (g.standard_normal((NR, D)) / np.sqrt(D)).astype(np.float32),
            "Proj": (g.standard_normal((NR, D, D)) / np.sqrt(D)).astype(np.float32),
            "dout": g.standard_normal(B).astype(np.float32),
            "h": g.integers(0, NE, B).astype(np.int32), "t": g.integers(0, NE, B).astype(np.int32), "r": g.integers(0, NR, B).astype(np.int32)}
    scal = {"batch_size": B, "dim": D, "nnodes": NE, "nedges": NR}
    out = {k: v for k, v in data.items()}
    tmp = tempfile.mkdtemp(prefix="program_golden_")
    for name, root in expressions(ns).items():
        transform.passes = [kge.fuser()]
        code = cpu.print_cpp(gen_ir(root))
        sig = re.search(r"torch::Tensor \w+\(([^)]*)\)\s*\{", code).group(1)
        order = [p.strip().split()[-1].replace("obj_", "") for p in sig.split(",")]
        path = os.path.join(tmp, f"{name}.cpp")
        open(path, "w").write(code)
        bdir = os.path.join(tmp, "build_" + name)
        os.makedirs(bdir)
        mod = load(name="prog_" + name, sources=[path], extra_cflags=["-O2"], build_directory=bdir, verbose=False)
        args = [scal[a] if a in scal else torch.from_numpy(data[a]) for a in order]
        res = mod.run(*args).numpy()
        out["out_" + name] = res
        out["args_" + name] = np.array(order)
        print(name, order, res.shape)
    np.savez_compressed(os.path.join(HERE, "program.npz"), **out)


if __name__ == "__main__":
    main()
