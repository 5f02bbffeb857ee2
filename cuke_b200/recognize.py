"""Recognises which KGE score function an expression graph states, and in which order its arguments are
passed to `run(...)`.

Recognition is structural: the graph is brought to a canonical form (sums flattened and sorted, commutative
products and dot products sorted, `apply` bodies reduced to their einsum/elementwise kind) and compared with
the canonical forms of the seven scorers written exactly as apps/kge/kge.py:273-390 writes them (DistMult and
ComplEx with the same operators), under every assignment of the user's tensors to the template's roles.

The positional order is that of cuke's helpers.get_input_nodes (pycuke1/helpers.py:179-190): post-order over
the graph, a node's size variables before its operands, each argument once; the three side tables of a
`reuse` index tensor directly after it.
"""
from __future__ import annotations

import itertools

from . import asg
from .asg import Const, Tensor, TensorOp, Var, _Item


# ---- positional argument order ---------------------------------------------------------------------------
def input_nodes(root):
    order, seen = [], set()

    def visit(n):
        if not isinstance(n, asg.ASTNode) or id(n) in seen:
            return
        seen.add(id(n))
        if isinstance(n, Const):
            return
        if isinstance(n, TensorOp):
            for s in n.ref_size:
                visit(s)
            for o in n.operators:
                visit(o)
            return
        if isinstance(n, _Item):
            return
        for s in n.ref_size:
            visit(s)
        if n.attr.get('is_arg'):
            order.append((n.name, n))
            if n.attr.get('reuse') and 'idx' in n.attr:
                for nm in n.attr['idx']:
                    order.append((nm, None))
    visit(root)
    return order


# ---- canonical form -----------------------------------------------------------------------------------------
def _key(c):
    return repr(c)


def canon(n, env=None):
    env = env or {}
    if isinstance(n, _Item):
        return env[id(n)]
    if isinstance(n, Const):
        return ('c', n.val)
    if isinstance(n, TensorOp):
        t = n.op_type
        if t in ('add', 'sub'):
            terms = []

            def flat(x, sign):
                if isinstance(x, TensorOp) and x.op_type in ('add', 'sub') and not isinstance(x, _Item):
                    flat(x.operators[0], sign)
                    flat(x.operators[1], sign if x.op_type == 'add' else -sign)
                else:
                    terms.append((sign, canon(x, env)))
            flat(n, 1)
            return ('sum', tuple(sorted(terms, key=_key)))
        if t == 'mul':
            fs = []

            def flatm(x):
                if isinstance(x, TensorOp) and x.op_type == 'mul':
                    flatm(x.operators[0]); flatm(x.operators[1])
                else:
                    fs.append(canon(x, env))
            flatm(n)
            return ('mul', tuple(sorted(fs, key=_key)))
        if t == 'index':
            return ('idx', canon(n.operators[0], env), canon(n.operators[1], env))
        if t == 'einsum':
            a, b, exp = n.operators
            ca, cb = canon(a, env), canon(b, env)
            if exp == 'i,i->':
                return ('dot', tuple(sorted((ca, cb), key=_key)))
            return ('einsum', exp, ca, cb)
        if t == 'apply':
            sub = dict(env)
            for it, d in zip(n.items, n.data):
                sub[id(it)] = canon(d, env)
            return canon(n.body, sub)      # batched op == its per-item body over the operands
        raise NotImplementedError(t)
    if isinstance(n, Var) or isinstance(n, Tensor):
        return ('t', n.name)
    raise TypeError(n)


def _rename(c, m):
    if isinstance(c, tuple):
        if len(c) == 2 and c[0] == 't':
            return ('t', m.get(c[1], c[1]))
        out = tuple(_rename(x, m) for x in c)
        if out and out[0] in ('sum', 'mul', 'dot'):
            return (out[0], tuple(sorted(out[1], key=_key)))
        return out
    return c


def _leaves(root):
    found, seen = [], set()

    def visit(n):
        if not isinstance(n, asg.ASTNode) or id(n) in seen:
            return
        seen.add(id(n))
        if isinstance(n, TensorOp):
            for o in n.operators:
                visit(o)
            if n.op_type == 'apply':
                visit(n.body)
        elif isinstance(n, _Item) or isinstance(n, Const):
            return
        elif isinstance(n, Tensor) and not isinstance(n, Var):
            found.append(n)
    visit(root)
    return found


# ---- templates: the score functions as the reference writes them -----------------------------------------------
def _ops():
    from . import kge
    return kge.bvv, kge.bsv, kge.bvm


def _templates():
    bvv, bsv, bvm = _ops()
    out = {}

    def common():
        nnodes, nedges, dim, batch = Var(name='nnodes'), Var(name='nedges'), Var(name='dim'), Var(name='batch_size')
        h = Tensor((batch,), dtype='int', name='h'); t = Tensor((batch,), dtype='int', name='t')
        r = Tensor((batch,), dtype='int', name='r')
        return nnodes, nedges, dim, batch, h, t, r

    nn, ne, d, b, h, t, r = common()
    E = Tensor((nn, d), name='Eemb'); R = Tensor((ne, d), name='Remb')
    out['TransE'] = E[h] - E[t] + R[r]                                     # apps/kge/kge.py:293
    nn, ne, d, b, h, t, r = common()
    E = Tensor((nn, d), name='Eemb'); R = Tensor((ne, d), name='Remb'); P = Tensor((ne, d), name='Pemb')
    out['TransH'] = E[h] - E[t] + R[r] - bsv(bvv(P[r], E[h] - E[t]), P[r])  # apps/kge/kge.py:317
    nn, ne, d, b, h, t, r = common()
    E = Tensor((nn, d), name='Eemb'); R = Tensor((ne, d), name='Remb'); M = Tensor((ne, d, d), name='Proj')
    out['TransR'] = bvm(E[h] - E[t], M[r]) + R[r]                           # apps/kge/kge.py:342
    nn, ne, d, b, h, t, r = common()
    E = Tensor((nn, d), name='Eemb'); R = Tensor((ne, d), name='Remb')
    out['TransF'] = bvv(E[h] + R[r], E[t]) + bvv(E[t] - R[r], E[h])        # apps/kge/kge.py:363
    nn, ne, d, b, h, t, r = common()
    E = Tensor((nn, d), name='Eemb'); M = Tensor((ne, d, d), name='Proj')
    out['RESCAL'] = bvv(bvm(E[h], M[r]), E[t])                              # apps/kge/kge.py:389
    nn, ne, d, b, h, t, r = common()
    E = Tensor((nn, d), name='Eemb'); R = Tensor((ne, d), name='Remb')
    out['DistMult'] = bvv(E[h] * R[r], E[t])
    nn, ne, d, b, h, t, r = common()
    Er = Tensor((nn, d), name='Ere'); Ei = Tensor((nn, d), name='Eim')
    Rr = Tensor((ne, d), name='Rre'); Ri = Tensor((ne, d), name='Rim')
    out['ComplEx'] = bvv(Er[h] * Rr[r] - Ei[h] * Ri[r], Er[t]) + bvv(Er[h] * Ri[r] + Ei[h] * Rr[r], Ei[t])
    return out


_template_cache = None


def recognise(root):
    """Returns (model, roles) with roles mapping template names (Eemb, Remb, Pemb, Proj, Ere, Eim, Rre, Rim, h, r, t)
    to the user's tensor names; raises NotImplementedError if the graph is not one of the seven scorers."""
    global _template_cache
    if _template_cache is None:
        _template_cache = {m: (canon(n), _leaves(n)) for m, n in _templates().items()}
    cu = canon(root)
    user = _leaves(root)

    def kind(x):
        return (x.dtype == 'int' or x.dtype.startswith('int'), len(x.ref_size))

    for model, (ct, tl) in _template_cache.items():
        if sorted(map(kind, tl)) != sorted(map(kind, user)):
            continue
        groups = {}
        for x in tl:
            groups.setdefault(kind(x), []).append(x.name)
        ugroups = {}
        for x in user:
            ugroups.setdefault(kind(x), []).append(x.name)
        keys = list(groups)
        for perms in itertools.product(*[itertools.permutations(ugroups[k]) for k in keys]):
            m = {}
            for k, perm in zip(keys, perms):
                for tname, uname in zip(groups[k], perm):
                    m[uname] = tname
            if _rename(cu, m) == ct:
                return model, {tname: uname for uname, tname in m.items()}
    raise NotImplementedError('this expression is not one of the KGE score functions the prebuilt kernels implement '
                              '(TransE, TransH, TransR, TransF, DistMult, RESCAL, ComplEx)')
