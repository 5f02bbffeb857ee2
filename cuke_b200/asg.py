"""Expression front-end with the surface of cuke's pycuke1.asg (pycuke1/asg.py:22-46,88-161,256-300):
Tensor / Var / Const / TensorOp, the arithmetic operators, `Tensor[idx]` (the indirect-index gather),
`apply`, `einsum`, `new_op`.

cuke lowers such a graph to loops and emits CUDA text.  Here the graph is only *recorded*: codegen.gpu
recognises which score function it states and run.gpu dispatches to the prebuilt kernels.  The node
classes therefore keep just what recognition and the positional argument order need: operators, result
sizes (`ref_size`) and attributes (`attr`, e.g. r.attr['reuse'] = True).
"""
from __future__ import annotations

import inspect

arith_op = {'add': '+', 'sub': '-', 'mul': '*', 'floordiv': '/', 'truediv': '/', 'mod': '%'}
elementwise_op = list(arith_op.keys())
func_op = ['apply']
other_op = ['einsum', 'index']


def new_op(func):
    """Decorator naming a user-defined operator (pycuke1/asg.py:22-27): the result carries attr['op_name']."""
    def wrapper_func(*args, **kwargs):
        res = func(*args, **kwargs)
        res.attr['op_name'] = func.__name__
        return res
    wrapper_func.__name__ = func.__name__
    return wrapper_func


class ASTNode:
    nuniq = 0

    def __init__(self):
        self.id = ASTNode.nuniq
        ASTNode.nuniq += 1
        self.attr = {}
        self.ref_by = []
        self.eval = None


def _as_size(s):
    if isinstance(s, ASTNode):
        return s
    if isinstance(s, int):
        return Const(s, 'int')
    raise TypeError('tensor dimensions must be int or a scalar int variable')


class Tensor(ASTNode):
    """Tensor(size, dtype='float', name=None) — pycuke1/asg.py:106-119."""

    def __init__(self, size, dtype='float', name=None):
        super().__init__()
        self.ref_size = [_as_size(s) for s in size]
        self.dtype = dtype
        self.name = name if name is not None else f'_t{self.id}'
        self.attr['is_arg'] = True

    def _size(self):
        return self.ref_size

    def __add__(self, other): return TensorOp('add', self, other)
    def __radd__(self, other): return TensorOp('add', other, self)
    def __sub__(self, other): return TensorOp('sub', self, other)
    def __rsub__(self, other): return TensorOp('sub', other, self)
    def __mul__(self, other): return TensorOp('mul', self, other)
    def __rmul__(self, other): return TensorOp('mul', other, self)
    def __truediv__(self, other): return TensorOp('truediv', self, other)
    def __floordiv__(self, other): return TensorOp('floordiv', self, other)

    def __getitem__(self, idx):
        """Tensor[idx] with an int tensor idx: the indirect-index gather (pycuke1/asg.py:154-156)."""
        return TensorOp('index', self, idx)

    def apply(self, func, axis=0, out_ofs=None, cond=None):
        return apply(func, (self,), [_as_size(axis)], out_ofs, cond)


class Var(Tensor):
    """Var(dtype='int', name=None) — a scalar argument (pycuke1/asg.py:256-258)."""

    def __init__(self, dtype='int', name=None):
        super().__init__([], dtype, name)


class Const(Var):
    """Const(val, dtype) — pycuke1/asg.py:262-285."""

    def __init__(self, val, dtype):
        super().__init__(dtype)
        self.val = val
        self.attr['is_arg'] = False


def _wrap(x):
    if isinstance(x, ASTNode):
        return x
    if isinstance(x, bool):
        raise TypeError('bool operand')
    if isinstance(x, int):
        return Const(x, 'int')
    if isinstance(x, float):
        return Const(x, 'float')
    return x


class TensorOp(Tensor):
    """TensorOp(op_type, *operators) — pycuke1/asg.py:289-586 (only the ops the KGE path uses)."""
    Types = func_op + elementwise_op + other_op

    def __init__(self, op_type, *operators):
        if op_type not in TensorOp.Types:
            raise NotImplementedError(f"operator '{op_type}' is outside the KGE scoring path")
        self.op_type = op_type
        self.operators = [_wrap(o) for o in operators]
        size, dtype = self._infer()
        super().__init__(size, dtype, None)
        self.attr['is_arg'] = False
        for o in self.operators:
            if isinstance(o, ASTNode):
                o.ref_by.append(self)

    def _infer(self):
        ops = self.operators
        if self.op_type in elementwise_op:
            a, b = ops
            big = a if len(a.ref_size) >= len(b.ref_size) else b
            dtype = 'float' if 'float' in (a.dtype, b.dtype) else a.dtype
            return list(big.ref_size), dtype
        if self.op_type == 'index':
            table, idx = ops
            if not isinstance(idx, Tensor) or len(idx.ref_size) != 1:
                raise NotImplementedError('only Tensor[int_tensor] gathers are on the KGE scoring path')
            return [idx.ref_size[0]] + list(table.ref_size[1:]), table.dtype
        if self.op_type == 'einsum':
            a, b, exp = ops
            lhs, out = exp.split('->')
            ia, ib = lhs.split(',')
            dims = {}
            for sub, t in ((ia, a), (ib, b)):
                for ch, s in zip(sub, t.ref_size):
                    dims.setdefault(ch, s)
            return [dims[ch] for ch in out], a.dtype
        if self.op_type == 'apply':
            func = ops[0]
            n = len(inspect.signature(func).parameters)
            data = ops[1:1 + n]
            items = [_Item(d) for d in data]
            body = func(*items)
            self.body = body
            self.items = items
            self.data = list(data)
            return [data[0].ref_size[0]] + list(body.ref_size), body.dtype
        raise NotImplementedError(self.op_type)


class _Item(Tensor):
    """One element (along axis 0) of an operand of `apply`, seen from inside the applied function."""

    def __init__(self, parent):
        super().__init__(list(parent.ref_size[1:]), parent.dtype, None)
        self.parent = parent
        self.attr['is_arg'] = False


def apply(func, data, axes=None, out_ofs=None, cond=None):
    """apply(func, data, axes=None, out_ofs=None, cond=None) — pycuke1/asg.py:38-46.  Only axis 0 without
    offsets/conditions occurs on the KGE scoring path."""
    assert callable(func)
    nparam = len(inspect.signature(func).parameters)
    assert len(data) == nparam
    axes = list(axes) if axes else []
    while len(axes) < nparam:
        axes.append(Const(0, 'int'))
    for ax in axes:
        if not (isinstance(ax, Const) and ax.val == 0):
            raise NotImplementedError('apply over an axis other than 0 is outside the KGE scoring path')
    if out_ofs is not None or cond is not None:
        raise NotImplementedError('apply with out_ofs / cond is outside the KGE scoring path')
    return TensorOp('apply', func, *data, *axes)


def einsum(exp: str, tensor1, tensor2):
    """einsum(exp, t1, t2) — pycuke1/asg.py:88-89."""
    return TensorOp('einsum', tensor1, tensor2, exp)
