"""compile_and_run(code, *args) with the reference's signature and positional convention
(pycuke1/run/gpu.py:4-19; call sites apps/kge/test_cuke.py:54,104,153,198,244).  Nothing is compiled: `code` is
the descriptor produced by codegen.gpu.print_cuda and the arguments are bound by position to one call into
the prebuilt library.  Returns what the reference's module.run returns: the (batch, dim) vector for
TransE/TransH/TransR, the (batch,) score for TransF/RESCAL (and DistMult/ComplEx)."""
import json

import torch

from ..scoring import Scorer


def compile_and_run(code, *args):
    try:
        desc = json.loads(code)
        assert desc.get("kge_b200") == 1
    except Exception as e:
        raise ValueError("`code` is not a descriptor produced by cuke_b200.codegen.gpu.print_cuda") from e
    names = desc["args"]
    if len(args) != len(names):
        raise TypeError(f"{desc['model']}: expected {len(names)} positional arguments ({', '.join(names)}), got {len(args)}")
    bound = dict(zip(names, args))
    roles = desc["roles"]
    get = lambda role: bound[roles[role]] if role in roles else None
    model = desc["model"]
    h, r, t = get("h"), get("r"), get("t")
    batch = bound.get("batch_size")
    if isinstance(batch, int) and batch != h.shape[0]:
        h, r, t = h[:batch], r[:batch], t[:batch]      # the reference computes the first batch_size triples
    if model == "ComplEx":
        # the reference-expressible ComplEx keeps real and imaginary parts in separate tables; the kernels use
        # interleaved rows, so interleave on the way in (layout change only)
        ent = torch.stack((get("Ere"), get("Eim")), dim=-1).reshape(get("Ere").shape[0], -1).contiguous()
        rel = torch.stack((get("Rre"), get("Rim")), dim=-1).reshape(get("Rre").shape[0], -1).contiguous()
        rel2 = None
    else:
        ent, rel = get("Eemb"), get("Remb")
        rel2 = get("Pemb") if model == "TransH" else get("Proj")
    return Scorer(model, ent, rel, rel2).ref_forward(h.contiguous(), r.contiguous(), t.contiguous())
