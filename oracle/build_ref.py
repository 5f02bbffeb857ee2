"""Build the reference's own CPU implementation of the KGE scoring path into oracle/_ref/.

TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Nothing in the shipped package may import this file
or anything it produces; only the tests, the smoke check and the benchmark's CPU-baseline /
reference legs do.

The reference (parallel-group/cuke) has no hand-written CPU scorer: its CPU path is C++ *text*
emitted by its own code generator.  This script imports that generator from the read-only
reference checkout, builds each score-function expression exactly as the reference's
apps/kge/kge.py:273-390 does (DistMult and ComplEx, which the reference does not ship, are
written with the same reference operators), lowers it with pycuke1.asg2ir.gen_ir, prints it
with pycuke1.codegen.cpu.print_cpp (pycuke1/codegen/cpu.py:110-150) and compiles the text
with torch.utils.cpp_extension.  Two variants per scorer:

  <name>       passes = [kge.fuser()]                      single thread; the parity oracle
  <name>_omp   passes = [kge.fuser(), outer parallelize]   `#pragma omp parallel for` on the batch
               loop (pycuke1/codegen/cpu.py:53-54); the timed CPU baseline.  The generated
               text references `tid0` without declaring it (pycuke1/transform/parallelize.py:242),
               so one line `const int tid0 = omp_get_thread_num();` is inserted at the top of
               each parallel loop body, and the `num_threads(N)` clause is clamped to the online
               cores; nothing else is touched.

Outputs go only to oracle/_ref/ (git-ignored; it travels to the GPU box as built files).
No reference source is copied: the .cpp files are outputs of running the reference.

  ref_transE_cuda  (--cuda-anchor) the reference's generated CUDA kernel for TransE without relation reuse, for sm_100:
                   the GPU-against-GPU anchor of the benchmark's side records.

Usage:  python oracle/build_ref.py [--ref <cuke checkout>] [--only transE,...] [--threads T] [--cuda-anchor]
"""
from __future__ import annotations

import argparse
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

SCORERS = ["transE", "transH", "transR", "transF", "RESCAL", "distmult", "complex"]

# Positional `run(...)` argument order of each generated module (post-order traversal of the
# expression graph, pycuke1/helpers.py:179-190); ids are int32 on the CPU path (codegen/cpu.py:90).
ARG_ORDER = {
    "transE": "batch_size, dim, nnodes, Eemb, h, t, nedges, Remb, r",
    "transH": "batch_size, dim, nnodes, Eemb, h, t, nedges, Remb, r, Pemb",
    "transR": "batch_size, dim, nnodes, Eemb, h, t, nedges, Proj, r, Remb",
    "transF": "batch_size, dim, nnodes, Eemb, h, nedges, Remb, r, t",
    "RESCAL": "batch_size, dim, nnodes, Eemb, h, nedges, Proj, r, t",
    "distmult": "batch_size, dim, nnodes, Eemb, h, nedges, Remb, r, t",
    "complex": "batch_size, dim, nnodes, Ere, h, nedges, Rre, r, Eim, Rim, t",
}


def _build_expr(name, ns):
    """Return the root node of scorer `name`, written with the reference's operators."""
    Var, Tensor = ns["Var"], ns["Tensor"]
    bvv, bsv, bvm = ns["bvv"], ns["bsv"], ns["bvm"]
    nnodes = Var(name="nnodes")
    nedges = Var(name="nedges")
    dim = Var(name="dim")
    batch_size = Var(name="batch_size")
    h = Tensor((batch_size,), dtype="int", name="h")
    t = Tensor((batch_size,), dtype="int", name="t")
    r = Tensor((batch_size,), dtype="int", name="r")
    if name == "complex":
        Ere = Tensor((nnodes, dim), name="Ere")
        Eim = Tensor((nnodes, dim), name="Eim")
        Rre = Tensor((nedges, dim), name="Rre")
        Rim = Tensor((nedges, dim), name="Rim")
        hr, hi, tr, ti, rr, ri = Ere[h], Eim[h], Ere[t], Eim[t], Rre[r], Rim[r]
        return bvv(hr * rr - hi * ri, tr) + bvv(hr * ri + hi * rr, ti)
    Eemb = Tensor((nnodes, dim), name="Eemb")
    if name == "transE":          # apps/kge/kge.py:273-293
        Remb = Tensor((nedges, dim), name="Remb")
        return Eemb[h] - Eemb[t] + Remb[r]
    if name == "transH":          # apps/kge/kge.py:296-318
        Remb = Tensor((nedges, dim), name="Remb")
        Pemb = Tensor((nedges, dim), name="Pemb")
        vh, vt, vr, vp = Eemb[h], Eemb[t], Remb[r], Pemb[r]
        return vh - vt + vr - bsv(bvv(vp, vh - vt), vp)
    if name == "transR":          # apps/kge/kge.py:321-343
        Remb = Tensor((nedges, dim), name="Remb")
        Proj = Tensor((nedges, dim, dim), name="Proj")
        vh, vt, mr, vr = Eemb[h], Eemb[t], Proj[r], Remb[r]
        return bvm(vh - vt, mr) + vr
    if name == "transF":          # apps/kge/kge.py:346-367
        Remb = Tensor((nedges, dim), name="Remb")
        vh, vt, vr = Eemb[h], Eemb[t], Remb[r]
        return bvv(vh + vr, vt) + bvv(vt - vr, vh)
    if name == "RESCAL":          # apps/kge/kge.py:370-390
        Proj = Tensor((nedges, dim, dim), name="Proj")
        vh, vt, mr = Eemb[h], Eemb[t], Proj[r]
        return bvv(bvm(vh, mr), vt)
    if name == "distmult":        # not in the reference; same operators
        Remb = Tensor((nedges, dim), name="Remb")
        return bvv(Eemb[h] * Remb[r], Eemb[t])
    raise KeyError(name)


def _patch_omp(code: str, threads: int) -> str:
    """Two textual patches, both confined to the OpenMP scaffolding of the generated text:
    (1) declare `tid0` at the top of every OpenMP-parallel batch loop body (the CPU back-end uses
    it without declaring it); (2) clamp the `num_threads(N)` clause to the online cores, because N
    also sizes the per-thread accumulator arrays and must stay the upper bound of `tid0`."""
    pat = re.compile(r"(#pragma omp parallel for[^\n]*\n\s*for \([^\n]*\)\s*\{\n)")
    code, n = pat.subn(lambda m: m.group(1) + "const int tid0 = omp_get_thread_num();\n", code)
    if n == 0:
        raise RuntimeError("no OpenMP batch loop found in generated code")
    code = code.replace(f"num_threads({threads})",
                        f"num_threads(omp_get_num_procs() < {threads} ? omp_get_num_procs() : {threads})")
    return "#include <omp.h>\n" + code


def generate(ref_root: str, names, threads: int):
    sys.path[:0] = [ref_root, os.path.join(ref_root, "apps", "kge")]
    os.environ["PYTHONDONTWRITEBYTECODE"] = "1"
    sys.dont_write_bytecode = True
    import kge  # noqa: the reference's apps/kge/kge.py
    from pycuke1 import transform
    from pycuke1.codegen import cpu
    from pycuke1.asg import Var, Tensor
    from pycuke1.asg2ir import gen_ir
    from pycuke1.helpers import ASGTraversal

    class outer_par:
        def __call__(self, node):
            def action(n, res):
                if "scope" not in n.attr and len(n.compute) > 0:
                    transform.parallelize.parallelize_loop(n, threads, [0])
            ASGTraversal(action)(node)
            return node

    ns = dict(Var=Var, Tensor=Tensor, bvv=kge.bvv, bsv=kge.bsv, bvm=kge.bvm)
    os.makedirs(OUT, exist_ok=True)
    made = []
    for name in names:
        for variant in ("", "_omp"):
            transform.passes = [kge.fuser()] + ([outer_par()] if variant else [])
            code = cpu.print_cpp(gen_ir(_build_expr(name, ns)))
            if variant:
                code = _patch_omp(code, threads)
            path = os.path.join(OUT, f"ref_{name}{variant}.cpp")
            with open(path, "w") as f:
                f.write(code)
            made.append((f"ref_{name}{variant}", path))
    return made


def compile_all(made):
    os.environ["CXX"] = "/usr/bin/g++"   # the image's default g++ has no libgomp.spec
    os.environ["CC"] = "/usr/bin/gcc"
    from torch.utils.cpp_extension import load
    for modname, path in made:
        bdir = os.path.join(OUT, "build_" + modname)
        os.makedirs(bdir, exist_ok=True)
        load(name=modname, sources=[path], extra_cflags=["-O2", "-fopenmp"],
             extra_ldflags=["-fopenmp"], build_directory=bdir, verbose=False)
        so = os.path.join(bdir, modname + ".so")
        if not os.path.exists(so):
            raise RuntimeError(f"{so} not produced")
        os.replace(so, os.path.join(OUT, modname + ".so"))
        print("built", modname, flush=True)


def generate_cuda_anchor(ref_root: str):
    """The reference's OWN GPU kernel for one scorer, as a GPU-against-GPU anchor: TransE without relation reuse, exactly as
    apps/kge/test_cuke.py:27-54 builds it, printed by pycuke1.codegen.gpu.print_cuda (pycuke1/codegen/gpu.py:182-236) under
    the reference's default pass list (apps/kge/kge.py:226) and compiled for sm_100.  Only this variant: it has no shared
    memory and no inspector, its index arithmetic stays inside the batch for batch % 16 == 0 (grid batch / 16, block
    32 x 16, rows 16 b .. 16 b + 15 per block)."""
    sys.path[:0] = [ref_root, os.path.join(ref_root, "apps", "kge")]
    sys.dont_write_bytecode = True
    import importlib
    import kge  # noqa
    importlib.reload(kge)                      # restores transform.passes to the reference's default GPU pass list
    from pycuke1.asg import Tensor, Var
    from pycuke1.asg2ir import gen_ir
    from pycuke1.codegen import gpu
    nnodes, nedges, dim, batch_size = Var(name="nnodes"), Var(name="nedges"), Var(name="dim"), Var(name="batch_size")
    Eemb, Remb = Tensor((nnodes, dim), name="Eemb"), Tensor((nedges, dim), name="Remb")
    h = Tensor((batch_size,), dtype="int", name="h"); t = Tensor((batch_size,), dtype="int", name="t")
    r = Tensor((batch_size,), dtype="int", name="r")
    code = gpu.print_cuda(gen_ir(Eemb[h] - Eemb[t] + Remb[r]))
    os.makedirs(OUT, exist_ok=True)
    path = os.path.join(OUT, "ref_transE_cuda.cu")
    with open(path, "w") as f:
        f.write(code)
    os.environ["CXX"], os.environ["CC"] = "/usr/bin/g++", "/usr/bin/gcc"
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"
    from torch.utils.cpp_extension import load
    bdir = os.path.join(OUT, "build_ref_transE_cuda")
    os.makedirs(bdir, exist_ok=True)
    load(name="ref_transE_cuda", sources=[path], build_directory=bdir, verbose=False)
    os.replace(os.path.join(bdir, "ref_transE_cuda.so"), os.path.join(OUT, "ref_transE_cuda.so"))
    print("built ref_transE_cuda", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("CUKE_REFERENCE", os.path.join(HERE, "..", "..", "reference")),
                    help="the cuke checkout (default: $CUKE_REFERENCE, else a directory `reference` beside this repository)")
    ap.add_argument("--only", default=",".join(SCORERS))
    ap.add_argument("--threads", type=int, default=256,
                    help="num_threads() written into the OpenMP pragma; OMP_NUM_THREADS / "
                         "omp_set_num_threads cannot raise it, the runtime clamps it to the cores")
    ap.add_argument("--cuda-anchor", action="store_true", help="also build the reference's generated TransE CUDA kernel (oracle/_ref/ref_transE_cuda.so)")
    ap.add_argument("--cuda-anchor-only", action="store_true")
    a = ap.parse_args()
    if not os.path.isdir(a.ref):
        print("reference checkout not present; keeping prebuilt oracle/_ref as is")
        return 0
    if not a.cuda_anchor_only:
        made = generate(a.ref, a.only.split(","), a.threads)
        compile_all(made)
    if a.cuda_anchor or a.cuda_anchor_only:
        generate_cuda_anchor(a.ref)
    return 0


if __name__ == "__main__":
    sys.exit(main())
