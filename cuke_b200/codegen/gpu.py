"""print_cuda stand-in (pycuke1/codegen/gpu.py:182-236).  cuke returns CUDA source text; here the returned
"code" is a one-line JSON descriptor which run.gpu.compile_and_run binds against the prebuilt library: the name of the
recognised score function (its hand-written kernels), or - for any other expression of the same operators - a register
program for the general evaluator (cuke_b200.program, kge_eval_program), plus the positional argument list."""
import json

from .. import program, recognize, transform


def print_cuda(node) -> str:
    for p in transform.passes:
        node = p(node)
    args = [name for name, _ in recognize.input_nodes(node)]
    try:
        model, roles = recognize.recognise(node)
    except NotImplementedError:
        return json.dumps({"kge_b200": 1, "model": "program", "program": program.compile_graph(node), "args": args})
    return json.dumps({"kge_b200": 1, "model": model, "roles": roles, "args": args})
