"""cuke's C++ back-end (pycuke1/codegen/cpu.py:110-150) has no counterpart here: the scoring path runs on the GPU only."""


def print_cpp(node):
    raise NotImplementedError("cuke_b200 has no CPU code path; use codegen.gpu.print_cuda")
