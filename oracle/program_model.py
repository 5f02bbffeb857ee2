"""numpy interpreter of the register programs that cuke_b200.program compiles (the semantics of kge_eval_program in
include/kge_b200.h).  TEST INFRASTRUCTURE, NOT PRODUCT CODE: tests/test_program.py uses it to check the compiler on the
CPU against outputs of the reference's own generated C++ for the same expressions (tests/golden/program_*.npz), and the
GPU tests compare the kernel with the same golden outputs."""
import numpy as np


def run(prog: dict, tables, ids, batch: int, dim: int) -> np.ndarray:
    f32 = np.float32
    v = [np.zeros((batch, dim), dtype=f32) for _ in range(max(prog["n_vreg"], 1))]
    s = [np.zeros(batch, dtype=f32) for _ in range(max(prog["n_sreg"], 1))]
    rows = np.arange(batch)
    for op, dst, a, b, c in prog["ops"]:
        if op == 0:
            v[dst] = tables[a][ids[b][:batch]].astype(f32)
        elif op in (1, 2, 3, 4):
            x, y = v[a], v[b]
            v[dst] = (x + y if op == 1 else x - y if op == 2 else x * y if op == 3 else x / y).astype(f32)
        elif op == 5:
            v[dst] = np.repeat(s[a][:, None], dim, 1).astype(f32)
        elif op == 6:
            s[dst] = np.einsum("bi,bi->b", v[a].astype(np.float64), v[b].astype(np.float64)).astype(f32)
        elif op in (7, 8, 9, 10):
            x, y = s[a], s[b]
            s[dst] = (x + y if op == 7 else x - y if op == 8 else x * y if op == 9 else x / y).astype(f32)
        elif op == 11:
            s[dst] = np.full(batch, np.array([a], dtype=np.int32).view(np.float32)[0], dtype=f32)
        elif op == 12:
            M = tables[b][ids[c][:batch]].astype(np.float64)
            v[dst] = np.einsum("bk,bkj->bj", v[a].astype(np.float64), M).astype(f32)
        elif op == 13:
            v[dst] = tables[a][ids[b][:batch]].astype(np.float64).sum(1).astype(f32)
        elif op == 14:
            M = tables[b][ids[c][:batch]].astype(np.float64)
            v[dst] = np.einsum("bkj,bj->bk", M, v[a].astype(np.float64)).astype(f32)
        elif op == 15:
            v[dst] = tables[a][rows].astype(f32)
        elif op == 16:
            s[dst] = tables[a][rows].astype(f32)
        else:
            raise ValueError(op)
    o = prog["out"]
    scale = s[o["s"]] if o["s"] >= 0 else np.ones(batch, dtype=f32)
    if o["kind"] == 0:
        return v[o["a"]]
    if o["kind"] == 1:
        return s[o["a"]]
    if o["kind"] == 2:
        return (scale[:, None, None] * v[o["a"]][:, :, None] * v[o["b"]][:, None, :]).astype(f32)
    return (scale[:, None, None] * tables[o["table"]][ids[o["ids"]][:batch]]).astype(f32)
