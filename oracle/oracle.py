"""Python face of the CPU oracle.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs import this module; the shipped
package (cuke_b200/) never does.

  - build()/lib(): compile oracle/kge_oracle.c with gcc into oracle/_build/ and bind it with ctypes.
  - ref_forward / scores / grads: the restated algorithm on numpy arrays.  Negatives are handled the way
    the reference handles them: flattened into a longer batch of ordinary triples
    (apps/kge/data/data_init.py:55-61), or, for chunk-shared negatives, with the index arithmetic of the
    reference's view formulation (apps/examples/examples.py:1434-1441: negative j of triple i is row
    (i // chunk) * n_neg + j of the chunk's negative list).
  - inspect(): numpy model of the sort+unique inspector (np.unique + stable argsort), bit-exact contract.
  - load_ref(name): the reference's own generated C++ compiled by oracle/build_ref.py, if present.
"""
from __future__ import annotations

import ctypes as C
import importlib.util
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
LIB_PATH = os.path.join(BUILD_DIR, "libkge_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")

MODELS = {"TransE": 0, "TransH": 1, "TransR": 2, "TransF": 3, "DistMult": 4, "RESCAL": 5, "ComplEx": 6}
VECTOR_MODELS = ("TransE", "TransH", "TransR")
REF_NAMES = {"TransE": "transE", "TransH": "transH", "TransR": "transR", "TransF": "transF",
             "DistMult": "distmult", "RESCAL": "RESCAL", "ComplEx": "complex"}

_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "kge_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        os.makedirs(BUILD_DIR, exist_ok=True)
        cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
        subprocess.run([cc, "-O2", "-shared", "-fPIC", "-o", LIB_PATH, src, "-lm"], check=True)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        fp, ip, dp, lp = (C.POINTER(C.c_float), C.POINTER(C.c_int), C.POINTER(C.c_double), C.POINTER(C.c_int64))
        _lib.ko_ref_forward.argtypes = [C.c_int, C.c_long, C.c_int, fp, ip, ip, fp, ip, fp, fp]
        _lib.ko_norm_scores.argtypes = [C.c_long, C.c_int, fp, fp]
        _lib.ko_grad.argtypes = [C.c_int, C.c_long, C.c_int, fp, ip, ip, fp, ip, fp, fp, dp, dp, dp]
        _lib.ko_legacy_inspect.argtypes = [lp, C.c_long, C.c_long, lp, lp, lp]
        for f in (_lib.ko_ref_forward, _lib.ko_norm_scores, _lib.ko_grad, _lib.ko_legacy_inspect):
            f.restype = None
    return _lib


def _f(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _i(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a, ty):
    return None if a is None else a.ctypes.data_as(C.POINTER(ty))


def ref_forward(model: str, E, R, P2, h, r, t) -> np.ndarray:
    """What the reference's generated code returns: (B, d) vector or (B,) scalar per triple."""
    E, R, P2, h, r, t = _f(E), _f(R), _f(P2), _i(h), _i(r), _i(t)
    B, d = h.shape[0], E.shape[1]
    out = np.empty((B, d) if model in VECTOR_MODELS else (B,), dtype=np.float32)
    lib().ko_ref_forward(MODELS[model], B, d, _p(E, C.c_float), _p(h, C.c_int), _p(t, C.c_int), _p(R, C.c_float),
                         _p(r, C.c_int), _p(P2, C.c_float), _p(out, C.c_float))
    return out


def flat_scores(model: str, E, R, P2, h, r, t) -> np.ndarray:
    """Scalar score of every (h, r, t): reference output, plus -||.||_2 for the vector-valued scorers."""
    if model not in VECTOR_MODELS:
        return ref_forward(model, E, R, P2, h, r, t)
    # the (B, d) vectors are an intermediate here: long flattened batches go through in blocks (per-triple arithmetic,
    # so the result does not depend on the blocking)
    h, r, t = np.asarray(h), np.asarray(r), np.asarray(t)
    B, blk = h.shape[0], 1 << 15
    sc = np.empty(B, dtype=np.float32)
    for lo in range(0, B, blk):
        out = ref_forward(model, E, R, P2, h[lo:lo + blk], r[lo:lo + blk], t[lo:lo + blk])
        part = np.empty(out.shape[0], dtype=np.float32)
        lib().ko_norm_scores(out.shape[0], out.shape[1], _p(out, C.c_float), _p(part, C.c_float))
        sc[lo:lo + blk] = part
    return sc


def flatten(h, r, t, neg, neg_mode: str, n_neg_head: int = 0, chunk: int = 0):
    """Negative triples as a flat list, in the order of the scorer's neg_score output.

    per_triple: neg (B, n_neg) -> triple (i, j) replaces the head if j < n_neg_head else the tail
    (apps/kge/data/data_init.py:55-61).  chunk_shared: neg (B // chunk, n_neg) -> triple i is paired with
    every row of its chunk's list (apps/examples/examples.py:1434-1441)."""
    h, r, t, neg = (np.asarray(x, dtype=np.int64) for x in (h, r, t, neg))
    B = h.shape[0]
    if neg_mode == "per_triple":
        n_neg = neg.shape[1]
        cand = neg
    elif neg_mode == "chunk_shared":
        n_neg = neg.shape[1]
        cand = neg[np.arange(B) // chunk]          # (B, n_neg)
    else:
        raise ValueError(neg_mode)
    hh = np.repeat(h[:, None], n_neg, 1)
    tt = np.repeat(t[:, None], n_neg, 1)
    rr = np.repeat(r[:, None], n_neg, 1)
    head_cols = np.arange(n_neg) < n_neg_head
    hh = np.where(head_cols[None, :], cand, hh)
    tt = np.where(head_cols[None, :], tt, cand)
    return hh.reshape(-1), rr.reshape(-1), tt.reshape(-1)


def scores(model: str, E, R, P2, h, r, t, neg=None, neg_mode: str = "none", n_neg_head: int = 0, chunk: int = 0):
    """(pos (B,), neg (B, n_neg) or None)."""
    pos = flat_scores(model, E, R, P2, h, r, t)
    if neg is None or neg_mode == "none":
        return pos, None
    fh, fr, ft = flatten(h, r, t, neg, neg_mode, n_neg_head, chunk)
    ns = flat_scores(model, E, R, P2, fh, fr, ft)
    return pos, ns.reshape(len(pos), -1)


def grads(model: str, E, R, P2, h, r, t, dpos, neg=None, dneg=None, neg_mode: str = "none", n_neg_head: int = 0,
          chunk: int = 0):
    """Dense float64 gradient tables (gE, gR, gP2) of sum(dpos * pos) + sum(dneg * neg)."""
    E, R, P2 = _f(E), _f(R), _f(P2)
    hs, rs, ts, ds = [np.asarray(h)], [np.asarray(r)], [np.asarray(t)], [np.asarray(dpos, dtype=np.float32)]
    if neg is not None and neg_mode != "none":
        fh, fr, ft = flatten(h, r, t, neg, neg_mode, n_neg_head, chunk)
        hs.append(fh); rs.append(fr); ts.append(ft); ds.append(np.asarray(dneg, dtype=np.float32).reshape(-1))
    fh, fr, ft = _i(np.concatenate(hs)), _i(np.concatenate(rs)), _i(np.concatenate(ts))
    fd = np.ascontiguousarray(np.concatenate(ds), dtype=np.float32)
    gE = np.zeros(E.shape, dtype=np.float64)
    gR = None if R is None else np.zeros(R.shape, dtype=np.float64)
    gP = None if P2 is None else np.zeros(P2.shape, dtype=np.float64)
    lib().ko_grad(MODELS[model], fh.shape[0], E.shape[1], _p(E, C.c_float), _p(fh, C.c_int), _p(ft, C.c_int),
                  _p(R, C.c_float), _p(fr, C.c_int), _p(P2, C.c_float), _p(fd, C.c_float),
                  _p(gE, C.c_double), _p(gR, C.c_double), _p(gP, C.c_double))
    return gE, gR, gP


def inspect(ids):
    """numpy model of the GPU inspector: (uniq int64, inverse int32, perm int32, seg int32 (n+1,))."""
    ids = np.asarray(ids).reshape(-1)
    n = ids.shape[0]
    uniq, inverse, counts = np.unique(ids, return_inverse=True, return_counts=True)
    perm = np.argsort(ids, kind="stable").astype(np.int32)
    seg = np.full(n + 1, n, dtype=np.int32)
    seg[: len(uniq)] = np.concatenate([[0], np.cumsum(counts)[:-1]]) if len(uniq) else []
    return uniq.astype(np.int64), inverse.reshape(-1).astype(np.int32), perm, seg


def legacy_inspect(rel, rel_num: int):
    rel = np.ascontiguousarray(rel, dtype=np.int64)
    n = rel.shape[0]
    uniq = np.zeros((n // 16, 16), dtype=np.int64)
    buf = np.zeros((n // 16, 16), dtype=np.int64)
    cnt = np.zeros((n // 16,), dtype=np.int64)
    lib().ko_legacy_inspect(_p(rel, C.c_int64), n, rel_num, _p(uniq, C.c_int64), _p(buf, C.c_int64), _p(cnt, C.c_int64))
    return uniq, buf, cnt


# ---- the reference's own generated C++ (built by oracle/build_ref.py) ---------------------------------
_ref_mods = {}


def have_ref(model: str, omp: bool = False) -> bool:
    return os.path.exists(os.path.join(REF_DIR, f"ref_{REF_NAMES[model]}{'_omp' if omp else ''}.so"))


def load_ref(model: str, omp: bool = False):
    name = f"ref_{REF_NAMES[model]}{'_omp' if omp else ''}"
    if name not in _ref_mods:
        import torch  # noqa: F401  (the generated modules are torch extensions)
        spec = importlib.util.spec_from_file_location(name, os.path.join(REF_DIR, name + ".so"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _ref_mods[name] = mod
    return _ref_mods[name]


def ref_run(model: str, E, R, P2, h, r, t, omp: bool = False):
    """Calls the reference-generated module with its positional convention (pycuke1/helpers.py:179-190).
    torch CPU tensors in, torch tensor out; ids int32.  ComplEx tables are de-interleaved for it."""
    import torch
    mod = load_ref(model, omp)
    B, d, ne = int(h.shape[0]), int(E.shape[1]), int(E.shape[0])
    nr = int((R if R is not None else P2).shape[0])
    h, r, t = (x.to(torch.int32).contiguous() for x in (h, r, t))
    if model == "TransE":
        return mod.run(B, d, ne, E, h, t, nr, R, r)
    if model == "TransH":
        return mod.run(B, d, ne, E, h, t, nr, R, r, P2)
    if model == "TransR":
        return mod.run(B, d, ne, E, h, t, nr, P2, r, R)
    if model in ("TransF", "DistMult"):
        return mod.run(B, d, ne, E, h, nr, R, r, t)
    if model == "RESCAL":
        return mod.run(B, d, ne, E, h, nr, P2, r, t)
    if model == "ComplEx":
        Ere, Eim = E[:, 0::2].contiguous(), E[:, 1::2].contiguous()
        Rre, Rim = R[:, 0::2].contiguous(), R[:, 1::2].contiguous()
        return mod.run(B, d // 2, ne, Ere, h, nr, Rre, r, Eim, Rim, t)
    raise KeyError(model)


def have_ref_cuda() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "ref_transE_cuda.so"))


def load_ref_cuda():
    """The reference's own generated CUDA kernel for TransE without relation reuse (oracle/build_ref.py --cuda-anchor):
    module.run(batch_size, dim, nnodes, Eemb, h, t, nedges, Remb, r) with CUDA float32 tables and int64 ids, batch a
    multiple of 16; returns the (batch, dim) vectors h - t + r."""
    name = "ref_transE_cuda"
    if name not in _ref_mods:
        import torch  # noqa: F401
        spec = importlib.util.spec_from_file_location(name, os.path.join(REF_DIR, name + ".so"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _ref_mods[name] = mod
    return _ref_mods[name]
