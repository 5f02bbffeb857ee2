"""Global pass list, as pycuke1.transform.passes (pycuke1/transform/__init__.py:10).  Passes are callables
node -> node run by codegen.gpu.print_cuda; the scheduling passes of apps/kge/kge.py are accepted and, except
for the reuse marking of indirect_smem, have nothing to do because scheduling is fixed in the kernels."""
passes = []
