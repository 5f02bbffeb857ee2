"""pycuke1/run/cpu.py:4-13 has no counterpart: there is no CPU fallback."""


def compile_and_run(code, *args):
    raise NotImplementedError("cuke_b200 has no CPU code path; use run.gpu.compile_and_run")
