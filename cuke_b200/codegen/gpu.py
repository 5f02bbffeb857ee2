"""print_cuda stand-in (pycuke1/codegen/gpu.py:182-236).  cuke returns CUDA source text; here the returned
"code" is a one-line JSON descriptor naming the recognised score function and the positional argument list,
which run.gpu.compile_and_run binds against the prebuilt library."""
import json

from .. import recognize, transform


def print_cuda(node) -> str:
    for p in transform.passes:
        node = p(node)
    model, roles = recognize.recognise(node)
    args = [name for name, _ in recognize.input_nodes(node)]
    return json.dumps({"kge_b200": 1, "model": model, "roles": roles, "args": args})
