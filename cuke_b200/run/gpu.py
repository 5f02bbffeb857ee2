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
    if desc["model"] == "program":
        return _run_program(desc["program"], bound)
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


def _run_program(prog, bound):
    """An expression outside the seven score functions: one launch of the general evaluator (kge_eval_program)."""
    import ctypes as C

    from .. import _lib
    tables = [bound[n] for n in prog["tables"]]
    ids = [bound[n] for n in prog["ids"]]
    for x in tables:
        if not (torch.is_tensor(x) and x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()):
            raise TypeError("the general evaluator takes contiguous float32 CUDA tensors")
    for x in ids:
        if not (torch.is_tensor(x) and x.is_cuda and x.dtype == ids[0].dtype and x.dtype in (torch.int32, torch.int64) and x.is_contiguous()):
            raise TypeError("index tensors must be contiguous int32 or int64 CUDA tensors of one dtype")
    dim = None
    for x, rank in zip(tables, prog["table_ranks"]):
        if rank >= 2:
            dim = int(x.shape[-1])
    if dim is None:
        raise ValueError("the expression has no vector operand")
    if ids:
        batch = int(ids[0].shape[0])
    else:
        batch = int(tables[0].shape[0])
    if isinstance(bound.get("batch_size"), int):
        batch = min(batch, bound["batch_size"])          # the reference computes the first batch_size elements
    o = prog["out"]
    shape = {0: (batch, dim), 1: (batch,), 2: (batch, dim, dim), 3: (batch, dim, dim)}[o["kind"]]
    out = torch.empty(shape, dtype=torch.float32, device=tables[0].device)
    kp = _lib.KgeProgram()
    kp.n_ops, kp.n_vreg, kp.n_sreg = len(prog["ops"]), prog["n_vreg"], prog["n_sreg"]
    kp.out_kind, kp.out_a, kp.out_b, kp.out_s, kp.out_table, kp.out_ids = o["kind"], o["a"], o["b"], o["s"], o["table"], o["ids"]
    for k, ins in enumerate(prog["ops"]):
        for q in range(5):
            kp.ops[k][q] = ins[q]
    tp = (C.c_void_p * max(len(tables), 1))(*[x.data_ptr() for x in tables])
    ip = (C.c_void_p * max(len(ids), 1))(*[x.data_ptr() for x in ids])
    bits = 64 if (ids and ids[0].dtype == torch.int64) else 32
    _lib.check(_lib.lib().kge_eval_program(C.byref(kp), dim, batch, tp, len(tables), ip, bits, len(ids), out.data_ptr(),
                                           torch.cuda.current_stream().cuda_stream))
    return out
