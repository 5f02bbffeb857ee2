"""The apps/kge surface of cuke (apps/kge/kge.py): batched operators, the pass objects, the inspector and the
score-function entry points, with the same names and call conventions."""
from __future__ import annotations

from . import transform
from .asg import Tensor, Var, apply, einsum, new_op
from .asg2ir import gen_ir
from .codegen import gpu
from .scoring import legacy_inspector


# ---- batched operators (apps/kge/kge.py:13-35) ----------------------------------------------------------
@new_op
def bvv(a, b):
    return apply(lambda x, y: einsum('i,i->', x, y), (a, b))


@new_op
def bsv(a, b):
    return apply(lambda x, y: x * y, (a, b))


@new_op
def bvm(a, b):
    return apply(lambda x, y: einsum('i,ij->j', x, y), (a, b))


@new_op
def bov(a, b):
    return apply(lambda x, y: einsum('i,j->ij', x, y), (a, b))


@new_op
def bsm(a, b):
    return apply(lambda x, y: einsum(',ij->ij', x, y), (a, b))


@new_op
def bmm(a, b):
    return apply(lambda x, y: einsum('ik,kj->j', x, y), (a, b))


# ---- passes (apps/kge/kge.py:86-224) -----------------------------------------------------------------------
class fuser:
    """Loop fusion (apps/kge/kge.py:86-100): fusion is a property of the prebuilt kernels; nothing to rewrite."""

    def __call__(self, node):
        return node


class tiler:
    """Tiling / thread mapping (apps/kge/kge.py:102-128): fixed inside the kernels; C and D are accepted."""

    def __init__(self, C, D):
        self.C, self.D = C, D

    def __call__(self, node):
        return node


class smem(tiler):
    """Shared-memory caching of temporaries (apps/kge/kge.py:130-188): registers / shared memory in the kernels."""


class indirect_smem(tiler):
    """Inspector-executor reuse (apps/kge/kge.py:190-224).  As in the reference, every index tensor marked
    attr['reuse'] = True gains the three side-table arguments <name>_uniq, <name>_buf, <name>_unique_cnt right
    after it in the positional list; the kernels deduplicate rows themselves and ignore their contents."""

    def __call__(self, node):
        from .recognize import input_nodes
        for name, n in input_nodes(node):
            if n is not None and n.attr.get('reuse') and isinstance(n, Tensor):
                n.attr['idx'] = [f'{name}_uniq', f'{name}_buf', f'{name}_unique_cnt']
        return node


transform.passes = [fuser(), tiler(16, 64), smem(16, 64), indirect_smem(16, 64)]   # apps/kge/kge.py:226


def inspector(r, rel_num, C=16):
    """inspector(r, rel_num, C=16) -> (uniq, buf, cnt) — apps/kge/kge.py:249-271."""
    return legacy_inspector(r, rel_num, C)


# ---- score functions (apps/kge/kge.py:273-390): each returns the descriptor print_cuda produces -----------------
def _args():
    nnodes, nedges = Var(name='nnodes'), Var(name='nedges')
    dim, batch_size = Var(name='dim'), Var(name='batch_size')
    h = Tensor((batch_size,), dtype='int', name='h')
    t = Tensor((batch_size,), dtype='int', name='t')
    r = Tensor((batch_size,), dtype='int', name='r')
    r.attr['reuse'] = True
    return nnodes, nedges, dim, batch_size, h, t, r


def transE():
    nnodes, nedges, dim, batch_size, h, t, r = _args()
    Eemb = Tensor((nnodes, dim), name='Eemb'); Remb = Tensor((nedges, dim), name='Remb')
    res = Eemb[h] - Eemb[t] + Remb[r]
    return gpu.print_cuda(gen_ir(res))


def transH():
    nnodes, nedges, dim, batch_size, h, t, r = _args()
    Eemb = Tensor((nnodes, dim), name='Eemb'); Remb = Tensor((nedges, dim), name='Remb')
    Pemb = Tensor((nedges, dim), name='Pemb')
    vh, vt, vr, vp = Eemb[h], Eemb[t], Remb[r], Pemb[r]
    res = vh - vt + vr - bsv(bvv(vp, vh - vt), vp)
    return gpu.print_cuda(gen_ir(res))


def transR():
    nnodes, nedges, dim, batch_size, h, t, r = _args()
    Eemb = Tensor((nnodes, dim), name='Eemb'); Remb = Tensor((nedges, dim), name='Remb')
    Proj = Tensor((nedges, dim, dim), name='Proj')
    vh, vt, mr, vr = Eemb[h], Eemb[t], Proj[r], Remb[r]
    res = bvm(vh - vt, mr) + vr
    return gpu.print_cuda(gen_ir(res))


def transF():
    nnodes, nedges, dim, batch_size, h, t, r = _args()
    Eemb = Tensor((nnodes, dim), name='Eemb'); Remb = Tensor((nedges, dim), name='Remb')
    vh, vt, vr = Eemb[h], Eemb[t], Remb[r]
    res = bvv(vh + vr, vt) + bvv(vt - vr, vh)
    return gpu.print_cuda(gen_ir(res))


def RESCAL():
    nnodes, nedges, dim, batch_size, h, t, r = _args()
    Eemb = Tensor((nnodes, dim), name='Eemb'); Proj = Tensor((nedges, dim, dim), name='Proj')
    vh, vt, mr = Eemb[h], Eemb[t], Proj[r]
    res = bvv(bvm(vh, mr), vt)
    return gpu.print_cuda(gen_ir(res))


def distmult():
    """Not in the reference; written with its operators."""
    nnodes, nedges, dim, batch_size, h, t, r = _args()
    Eemb = Tensor((nnodes, dim), name='Eemb'); Remb = Tensor((nedges, dim), name='Remb')
    res = bvv(Eemb[h] * Remb[r], Eemb[t])
    return gpu.print_cuda(gen_ir(res))


def complEx():
    """Not in the reference; split real/imaginary tables, the only complex form its operators can state."""
    nnodes, nedges, dim, batch_size, h, t, r = _args()
    Ere = Tensor((nnodes, dim), name='Ere'); Eim = Tensor((nnodes, dim), name='Eim')
    Rre = Tensor((nedges, dim), name='Rre'); Rim = Tensor((nedges, dim), name='Rim')
    hr, hi, tr, ti, rr, ri = Ere[h], Eim[h], Ere[t], Eim[t], Rre[r], Rim[r]
    res = bvv(hr * rr - hi * ri, tr) + bvv(hr * ri + hi * rr, ti)
    return gpu.print_cuda(gen_ir(res))
