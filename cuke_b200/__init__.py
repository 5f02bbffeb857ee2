"""cuke_b200 — KGE scoring (cuke's apps/kge hot path) on NVIDIA B200 behind cuke's operator surface.

    from cuke_b200.asg import *; from cuke_b200 import kge, run, transform
    code = gpu.print_cuda(gen_ir(expr));  out = run.gpu.compile_and_run(code, *args)

or, to run an unmodified cuke script, `cuke_b200.install_as_pycuke1()` registers this package under the names
`pycuke1`, `pycuke1.asg`, ... and `kge`.
"""
import sys

__version__ = "0.1.0"


def install_as_pycuke1() -> None:
    """Makes `import pycuke1`, `from pycuke1.asg import *`, `import kge` resolve to this package."""
    from . import asg, asg2ir, codegen, kge, run, transform
    pkg = sys.modules[__name__]
    sys.modules.setdefault("pycuke1", pkg)
    for name, mod in (("asg", asg), ("asg2ir", asg2ir), ("codegen", codegen), ("run", run), ("transform", transform)):
        sys.modules.setdefault(f"pycuke1.{name}", mod)
    sys.modules.setdefault("pycuke1.codegen.gpu", codegen.gpu)
    sys.modules.setdefault("pycuke1.codegen.cpu", codegen.cpu)
    sys.modules.setdefault("pycuke1.run.gpu", run.gpu)
    sys.modules.setdefault("pycuke1.run.cpu", run.cpu)
    sys.modules.setdefault("kge", kge)
