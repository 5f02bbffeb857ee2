"""Compiler from an expression graph of the reference's batched operators to a register program for kge_eval_program.

cuke generates a kernel for any composition of its operators over gathered rows (what its fusion rule covers is listed in
apps/kge/kge.py:36-84).  The seven score functions are recognised structurally (cuke_b200.recognize) and run on
hand-written kernels; everything else lands here: the graph is walked once per batch element - `apply` is transparent,
because the evaluator already works element by element - and every node becomes an instruction over per-element vector
registers (length dim), scalar registers, or a restricted matrix value (a gathered (dim, dim) row, an outer product, or
either times a scalar), which may only be consumed by a vector-matrix product or be the result.

Supported: Tensor[int_tensor] gathers from (n, dim) and (n, dim, dim) tables; (batch, dim) and (batch,) float operands
used element by element; + - * / between vectors, scalars (broadcast) and constants; einsum 'i,i->' (bvv), 'i,ij->j'
(bvm), 'ij,j->i', 'i,j->ij' (bov), ',ij->ij' (bsm), 'ik,kj->j' (bmm); apply over axis 0.
"""
from __future__ import annotations

import struct
from typing import Dict, List, Tuple

from . import asg
from .asg import Const, Tensor, TensorOp, Var, _Item

OPS = {"GATHER": 0, "VADD": 1, "VSUB": 2, "VMUL": 3, "VDIV": 4, "SPLAT": 5, "DOT": 6, "SADD": 7, "SSUB": 8, "SMUL": 9, "SDIV": 10,
       "SCONST": 11, "VECMAT": 12, "COLSUM": 13, "MATVEC": 14, "ROW": 15, "LOADS": 16}
OUT_VECTOR, OUT_SCALAR, OUT_OUTER, OUT_MATRIX = 0, 1, 2, 3
_V = {"add": "VADD", "sub": "VSUB", "mul": "VMUL", "truediv": "VDIV"}
_S = {"add": "SADD", "sub": "SSUB", "mul": "SMUL", "truediv": "SDIV"}
# which operand fields of an instruction name vector / scalar registers: (dst kind, kinds of a, b)
_REGS = {"GATHER": ("v", "", ""), "VADD": ("v", "v", "v"), "VSUB": ("v", "v", "v"), "VMUL": ("v", "v", "v"), "VDIV": ("v", "v", "v"),
         "SPLAT": ("v", "s", ""), "DOT": ("s", "v", "v"), "SADD": ("s", "s", "s"), "SSUB": ("s", "s", "s"), "SMUL": ("s", "s", "s"),
         "SDIV": ("s", "s", "s"), "SCONST": ("s", "", ""), "VECMAT": ("v", "v", ""), "COLSUM": ("v", "", ""), "MATVEC": ("v", "v", ""),
         "ROW": ("v", "", ""), "LOADS": ("s", "", "")}


class _Builder:
    def __init__(self):
        self.code: List[list] = []          # [op name, dst, a, b, c] over virtual registers
        self.tables: List[Tensor] = []
        self.ids: List[Tensor] = []
        self.nv = self.ns = 0
        self.memo: Dict[tuple, tuple] = {}

    def table(self, t: Tensor) -> int:
        for k, x in enumerate(self.tables):
            if x is t:
                return k
        self.tables.append(t)
        return len(self.tables) - 1

    def idarr(self, t: Tensor) -> int:
        for k, x in enumerate(self.ids):
            if x is t:
                return k
        self.ids.append(t)
        return len(self.ids) - 1

    def emit(self, op, a=0, b=0, c=0):
        kind = _REGS[op][0]
        if kind == "v":
            dst, self.nv = self.nv, self.nv + 1
        else:
            dst, self.ns = self.ns, self.ns + 1
        self.code.append([op, dst, a, b, c])
        return (kind, dst)

    # ---- walk ------------------------------------------------------------------------------------------------------
    def val(self, n, env):
        if not isinstance(n, _Item) and id(n) in self.memo:
            return self.memo[id(n)]
        out = self._val(n, env)
        if not isinstance(n, _Item) and not env:
            self.memo[id(n)] = out
        return out

    def _val(self, n, env):
        if isinstance(n, _Item):
            return env[id(n)]
        if isinstance(n, Const):
            bits = struct.unpack("<i", struct.pack("<f", float(n.val)))[0]
            return self.emit("SCONST", bits)
        if isinstance(n, TensorOp):
            return self._op(n, env)
        if isinstance(n, Var):
            raise NotImplementedError(f"scalar argument {n.name} inside an expression")
        if isinstance(n, Tensor):
            if n.dtype == "int" or str(n.dtype).startswith("int"):
                raise NotImplementedError(f"{n.name}: an index tensor can only be used as Tensor[index]")
            rank = len(n.ref_size)
            if rank == 1:
                return self.emit("LOADS", self.table(n))
            if rank == 2:
                return self.emit("ROW", self.table(n))
            raise NotImplementedError(f"{n.name}: a rank-{rank} operand must be gathered through an index tensor")
        raise TypeError(n)

    def _as_vector(self, x):
        if x[0] == "v":
            return x
        if x[0] == "s":
            return self.emit("SPLAT", x[1])
        raise NotImplementedError("a matrix value where a vector is needed")

    def _op(self, n, env):
        t = n.op_type
        if t == "index":
            table, idx = n.operators
            if not (isinstance(table, Tensor) and not isinstance(table, TensorOp) and isinstance(idx, Tensor) and not isinstance(idx, TensorOp)):
                raise NotImplementedError("gathers must be argument_tensor[argument_index_tensor]")
            rank = len(table.ref_size)
            if rank == 2:
                key = ("gather", id(table), id(idx))          # the same row gathered twice is one instruction
                if key not in self.memo:
                    self.memo[key] = self.emit("GATHER", self.table(table), self.idarr(idx))
                return self.memo[key]
            if rank == 3:
                return ("m", ("gather", self.table(table), self.idarr(idx)))
            raise NotImplementedError(f"gather from a rank-{rank} table")
        if t in _V:
            a, b = (self.val(o, env) for o in n.operators)
            if a[0] == "s" and b[0] == "s":
                return self.emit(_S[t], a[1], b[1])
            if "m" in (a[0], b[0]):
                if t == "mul" and {a[0], b[0]} == {"m", "s"}:
                    s, m = (a, b) if a[0] == "s" else (b, a)
                    return ("m", ("smat", s[1], m[1]))
                raise NotImplementedError("matrix values only support scalar * matrix")
            a, b = self._as_vector(a), self._as_vector(b)
            return self.emit(_V[t], a[1], b[1])
        if t == "einsum":
            xa, xb, exp = n.operators
            a, b = self.val(xa, env), self.val(xb, env)
            if exp == "i,i->":
                return self.emit("DOT", self._as_vector(a)[1], self._as_vector(b)[1])
            if exp == "i,ij->j":
                if b[0] != "m" or b[1][0] != "gather":
                    raise NotImplementedError("'i,ij->j' needs a gathered (dim, dim) matrix as its second operand")
                return self.emit("VECMAT", self._as_vector(a)[1], b[1][1], b[1][2])
            if exp == "ij,j->i":
                if a[0] != "m" or a[1][0] != "gather":
                    raise NotImplementedError("'ij,j->i' needs a gathered (dim, dim) matrix as its first operand")
                return self.emit("MATVEC", self._as_vector(b)[1], a[1][1], a[1][2])
            if exp == "i,j->ij":
                return ("m", ("outer", self._as_vector(a)[1], self._as_vector(b)[1]))
            if exp == ",ij->ij":
                if a[0] != "s" or b[0] != "m":
                    raise NotImplementedError("',ij->ij' needs a scalar and a matrix")
                return ("m", ("smat", a[1], b[1]))
            if exp == "ik,kj->j":
                if a[0] != "m" or a[1][0] != "gather" or b[0] != "m" or b[1][0] != "gather":
                    raise NotImplementedError("'ik,kj->j' needs two gathered matrices")
                u = self.emit("COLSUM", a[1][1], a[1][2])
                return self.emit("VECMAT", u[1], b[1][1], b[1][2])
            raise NotImplementedError(f"einsum '{exp}'")
        if t == "apply":
            sub = dict(env)
            for it, d in zip(n.items, n.data):
                sub[id(it)] = self.val(d, env)
            return self.val(n.body, sub)
        raise NotImplementedError(t)


def _allocate(code, result_regs):
    """Linear scan over the virtual registers: a physical register is free again after its value's last use."""
    last = {}
    for pc, (op, dst, a, b, c) in enumerate(code):
        kinds = _REGS[op]
        for kind, r in ((kinds[1], a), (kinds[2], b)):
            if kind:
                last[(kind, r)] = pc
    for kr in result_regs:
        last[kr] = len(code)
    phys, free, count = {}, {"v": [], "s": []}, {"v": 0, "s": 0}
    out = []
    for pc, (op, dst, a, b, c) in enumerate(code):
        kinds = _REGS[op]
        pa = phys[(kinds[1], a)] if kinds[1] else a
        pb = phys[(kinds[2], b)] if kinds[2] else b
        released = []
        for kind, r in ((kinds[1], a), (kinds[2], b)):
            if kind and last.get((kind, r)) == pc and (kind, r) not in released:
                released.append((kind, r))
        # matrix-vector products must not write over their vector operand: release operands only after the destination is chosen
        k = kinds[0]
        if op not in ("VECMAT", "MATVEC"):         # element-wise: the destination may take over an operand's register
            for kr in released:
                free[kr[0]].append(phys[kr])
            released = []
        if free[k]:
            pd = free[k].pop()
        else:
            pd, count[k] = count[k], count[k] + 1
        phys[(k, dst)] = pd
        for kr in released:
            free[kr[0]].append(phys[kr])
        if last.get((k, dst)) is None:             # never read: free at once
            free[k].append(pd)
        out.append([OPS[op], pd, pa, pb, c])
    return out, phys, max(count["v"], 0), max(count["s"], 0)


def compile_graph(root) -> dict:
    """Returns the program as a JSON-able dict: ops, register counts, result, and the names of the table and id-array
    arguments in the order the program numbers them."""
    b = _Builder()
    res = b.val(root, {})
    result_regs = []
    out = {"kind": None, "a": 0, "b": 0, "s": -1, "table": 0, "ids": 0}
    if res[0] == "v":
        out["kind"], out["a"] = OUT_VECTOR, ("v", res[1]); result_regs.append(("v", res[1]))
    elif res[0] == "s":
        out["kind"], out["a"] = OUT_SCALAR, ("s", res[1]); result_regs.append(("s", res[1]))
    else:
        form, scal = res[1], None
        while form[0] == "smat":
            if scal is None:
                scal = ("s", form[1])
            else:
                scal = b.emit("SMUL", scal[1], form[1])
            form = form[2]
        if scal is not None:
            out["s"] = scal; result_regs.append(scal)
        if form[0] == "outer":
            out["kind"], out["a"], out["b"] = OUT_OUTER, ("v", form[1]), ("v", form[2])
            result_regs += [("v", form[1]), ("v", form[2])]
        else:
            out["kind"], out["table"], out["ids"] = OUT_MATRIX, form[1], form[2]
    if len(b.code) > 64:
        raise NotImplementedError(f"the expression needs {len(b.code)} instructions (limit 64)")
    ops, phys, nv, ns = _allocate(b.code, result_regs)
    for k in ("a", "b", "s"):
        if isinstance(out[k], tuple):
            out[k] = phys[out[k]]
    if nv > 16 or ns > 16 or len(b.tables) > 8 or len(b.ids) > 4:
        raise NotImplementedError("the expression exceeds the evaluator's limits (16 vector / 16 scalar registers, 8 tables, 4 id arrays)")
    return {"ops": ops, "n_vreg": nv, "n_sreg": ns, "out": out, "tables": [t.name for t in b.tables], "ids": [t.name for t in b.ids],
            "table_ranks": [len(t.ref_size) for t in b.tables]}
