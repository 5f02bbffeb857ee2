"""Torch-facing wrappers over the C ABI: scorers, inspector, staging, segmented reduction.

PyTorch is used for device memory, streams and dtype bookkeeping only; every computation below is a call
into libkge_b200.so on the current CUDA stream.  All tensors must live on the current CUDA device.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import (DTYPES, MATRIX_MODELS, MODELS, NEG_MODES, PRECISIONS, VECTOR_MODELS, KgeGrads, KgeProblem, KgeTensors,
                   check)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(device=None) -> int:
    """Handle of the current CUDA stream of `device` (default: the current device).  The raw query is an order of
    magnitude cheaper than building a torch.cuda.Stream object, and a step makes dozens of these calls."""
    if _raw_stream is not None:
        idx = torch.cuda.current_device() if device is None or device.index is None else device.index
        return _raw_stream(idx)
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dtype_of(t: torch.Tensor) -> str:
    if t.dtype == torch.float32:
        return "f32"
    if t.dtype == torch.bfloat16:
        return "bf16"
    raise TypeError(f"tables must be float32 or bfloat16, got {t.dtype}")


def _id_bits(t: torch.Tensor) -> int:
    if t.dtype == torch.int64:
        return 64
    if t.dtype == torch.int32:
        return 32
    raise TypeError(f"ids must be int64 or int32, got {t.dtype}")


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not (t.is_cuda and t.is_contiguous()):
            raise ValueError("expected contiguous CUDA tensors")


_ws_cache = {}


def workspace(nbytes: int, device, tag: str = "") -> torch.Tensor:
    """A reusable scratch buffer per (device, current stream, tag); grown on demand, never shrunk.  Keyed by stream
    so that calls issued on different streams never share scratch."""
    key = (device.index if isinstance(device, torch.device) else str(device), _stream(device if isinstance(device, torch.device) else None), tag)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf


# ---- inspector ---------------------------------------------------------------------------------------------
@dataclass
class Inspection:
    """Result of the GPU inspector over an id list (see kge_inspect in include/kge_b200.h)."""
    uniq: torch.Tensor       # (n,) int64, first U entries valid
    inverse: torch.Tensor    # (n,) int32
    perm: torch.Tensor       # (n,) int32
    seg: torch.Tensor        # (n+1,) int32
    n_unique: torch.Tensor   # (1,) int64 on the device
    n: int

    def count(self) -> int:
        """U on the host (synchronises)."""
        return int(self.n_unique.item())


def inspect(ids: torch.Tensor, id_space: int) -> Inspection:
    _need_cuda(ids)
    ids = ids.reshape(-1)
    n = ids.numel()
    dev = ids.device
    uniq = torch.empty(max(n, 1), dtype=torch.int64, device=dev)
    inverse = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    perm = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    seg = torch.empty(n + 1, dtype=torch.int32, device=dev)
    n_unique = torch.empty(1, dtype=torch.int64, device=dev)
    L = _lib.lib()
    need = L.kge_inspect_workspace_bytes(n)
    ws = workspace(need, dev, "inspect")
    check(L.kge_inspect(_ptr(ids), _id_bits(ids), n, int(id_space), _ptr(ws), ws.numel(), _ptr(uniq), _ptr(inverse),
                        _ptr(perm), _ptr(seg), _ptr(n_unique), _stream()))
    return Inspection(uniq, inverse, perm, seg, n_unique, n)


def legacy_inspector(r: torch.Tensor, rel_num: int, C_: int = 16):
    """Drop-in for the reference's `inspector(r, rel_num, C=16)` (apps/kge/kge.py:249-271)."""
    if C_ != 16:
        raise ValueError("the reference inspector is compiled for C = 16 (apps/kge/inspection/inspector.cu:10)")
    _need_cuda(r)
    if r.dtype != torch.int64:
        raise TypeError("relation ids must be int64 (the reference's GPU convention)")
    n = r.shape[0] // 16 * 16
    uniq = torch.zeros((r.shape[0] // 16, 16), dtype=torch.int64, device=r.device)
    buf = torch.zeros((r.shape[0] // 16, 16), dtype=torch.int64, device=r.device)
    cnt = torch.zeros((r.shape[0] // 16,), dtype=torch.int64, device=r.device)
    check(_lib.lib().kge_legacy_inspect(_ptr(r), n, int(rel_num), _ptr(uniq), _ptr(buf), _ptr(cnt), _stream()))
    return uniq, buf, cnt


def gather_rows(table: torch.Tensor, ids: torch.Tensor, n_dev: Optional[torch.Tensor] = None, first_row: int = 0,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = table[ids[i] - first_row] for i < min(len(ids), *n_dev): the dedup staging copy."""
    _need_cuda(table, ids, n_dev)
    n, dim = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty((n, dim), dtype=table.dtype, device=table.device)
    check(_lib.lib().kge_gather_rows(_ptr(table), DTYPES[_dtype_of(table)], dim, _ptr(ids), n, _ptr(n_dev), int(first_row),
                                     _ptr(out), _stream()))
    return out


def scatter_rows(rows: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, n_dev: Optional[torch.Tensor] = None,
                 first_row: int = 0) -> torch.Tensor:
    """out[ids[i] - first_row] = rows[i] for i < min(len(ids), *n_dev); ids distinct."""
    _need_cuda(rows, ids, out, n_dev)
    check(_lib.lib().kge_scatter_rows(_ptr(rows), rows.shape[1], _ptr(ids), min(ids.numel(), rows.shape[0]), _ptr(n_dev),
                                      int(first_row), _ptr(out), _stream()))
    return out


def fma_peak_tflops(device=None, iters: int = 4096) -> float:
    """Attainable fp32 FMA rate of the current GPU in TFLOP/s (2 flops per FMA), from the library's probe kernel."""
    dev = device or torch.device("cuda", torch.cuda.current_device())
    out = torch.zeros(4, dtype=torch.float32, device=dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    flops = C.c_double(0.0)
    L = _lib.lib()
    check(L.kge_probe_fma(_ptr(out), sms * 8, 64, C.byref(flops), _stream()))
    torch.cuda.synchronize()
    best = 0.0
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        check(L.kge_probe_fma(_ptr(out), sms * 8, iters, C.byref(flops), _stream()))
        e1.record()
        torch.cuda.synchronize()
        best = max(best, flops.value / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return best


def segment_reduce(rows: torch.Tensor, insp: Inspection, out: Optional[torch.Tensor] = None,
                   n_out: Optional[int] = None, zero_tail: bool = True) -> torch.Tensor:
    """One fp32 row per distinct id: out[u] = sum of rows[slot] over the slots holding uniq[u] (fixed order).
    Rows of `out` past the number of distinct ids are zero-filled unless zero_tail is False."""
    _need_cuda(rows)
    n, dim = rows.shape
    if n != insp.n:
        raise ValueError(f"rows has {n} slots, the inspection {insp.n}")
    if out is None:
        out = torch.empty((n if n_out is None else n_out, dim), dtype=torch.float32, device=rows.device)
    L = _lib.lib()
    need = L.kge_segment_reduce_workspace_bytes(n, dim)
    ws = workspace(need, rows.device, "segred")
    check(L.kge_segment_reduce(_ptr(rows), dim, n, _ptr(insp.perm), _ptr(insp.seg), _ptr(insp.n_unique), _ptr(out),
                               out.shape[0] if zero_tail else 0, _ptr(ws), ws.numel(), _stream()))
    return out


def segment_reduce_static(rows: torch.Tensor, insp: Inspection, out: torch.Tensor) -> torch.Tensor:
    """segment_reduce through the entry point that owns its scratch: nothing is allocated, so `out` must be given.
    Limited to ceil(n/32) * dim <= 1,048,576; calls on one device must not overlap (they share the scratch)."""
    _need_cuda(rows, out)
    n, dim = rows.shape
    if n != insp.n:
        raise ValueError(f"rows has {n} slots, the inspection {insp.n}")
    check(_lib.lib().kge_segment_reduce_static(_ptr(rows), dim, n, _ptr(insp.perm), _ptr(insp.seg), _ptr(insp.n_unique),
                                               _ptr(out), out.shape[0], _stream()))
    return out


def apply_sgd(table: torch.Tensor, grad_rows: torch.Tensor, lr: float, ids: Optional[torch.Tensor] = None,
              n_dev: Optional[torch.Tensor] = None, first_row: int = 0) -> None:
    """table[ids[i] - first_row] -= lr * grad_rows[i] for i < min(len, *n_dev); ids distinct (None: row i)."""
    _need_cuda(table, grad_rows, ids, n_dev)
    n = grad_rows.shape[0] if ids is None else min(ids.numel(), grad_rows.shape[0])
    check(_lib.lib().kge_apply_sgd(_ptr(table), DTYPES[_dtype_of(table)], table.shape[1], _ptr(ids), n, _ptr(n_dev), int(first_row),
                                   _ptr(grad_rows), float(lr), _stream()))


def apply_adagrad(table: torch.Tensor, state: torch.Tensor, grad_rows: torch.Tensor, lr: float, eps: float = 1e-10,
                  ids: Optional[torch.Tensor] = None, n_dev: Optional[torch.Tensor] = None, first_row: int = 0) -> None:
    """Adagrad on the touched rows: state += g^2, table -= lr * g / (sqrt(state) + eps); state is fp32, shaped like table."""
    _need_cuda(table, state, grad_rows, ids, n_dev)
    if state.shape != table.shape or state.dtype != torch.float32:
        raise ValueError("state must be float32 with the table's shape")
    n = grad_rows.shape[0] if ids is None else min(ids.numel(), grad_rows.shape[0])
    check(_lib.lib().kge_apply_adagrad(_ptr(table), DTYPES[_dtype_of(table)], _ptr(state), table.shape[1], _ptr(ids), n, _ptr(n_dev),
                                       int(first_row), _ptr(grad_rows), float(lr), float(eps), _stream()))


def owner_counts(insp: Inspection, rows_per_rank: int, world: int) -> torch.Tensor:
    counts = torch.empty(world, dtype=torch.int64, device=insp.uniq.device)
    check(_lib.lib().kge_owner_counts(_ptr(insp.uniq), _ptr(insp.n_unique), insp.n, int(rows_per_rank), int(world),
                                      _ptr(counts), _stream()))
    return counts


def validate_ids(ids: torch.Tensor, id_space: int, sanitized: Optional[torch.Tensor] = None) -> None:
    """Range check of an id tensor (kge_validate_ids): ids outside [0, id_space) set ERR_ID_RANGE in the device error
    word (read it with device_flags()); `sanitized` (same shape and dtype, may be `ids`) receives the ids with 0 in
    place of the bad ones."""
    _need_cuda(ids, sanitized)
    if sanitized is not None and (sanitized.dtype != ids.dtype or sanitized.numel() != ids.numel()):
        raise ValueError("sanitized must match ids in dtype and size")
    check(_lib.lib().kge_validate_ids(_ptr(ids), _id_bits(ids), ids.numel(), int(id_space), _ptr(sanitized), _stream()))


def selftest_wait_timeout(polls: int = 2048) -> None:
    """Launches the library's wait self-test: a bounded wait that nothing completes runs out and reports ERR_WAIT_TIMEOUT."""
    check(_lib.lib().kge_selftest_wait_timeout(int(polls), _stream()))


def device_flags() -> int:
    """Reads and clears the device error word (synchronises the current stream); 0 = clean, else an OR of
    _lib.ERR_WAIT_TIMEOUT (a bounded wait inside a tensor-core kernel ran out: its outputs are invalid) and
    _lib.ERR_ID_RANGE (an id outside its table was met by a checked call)."""
    flags = C.c_int32(0)
    check(_lib.lib().kge_check(_stream(), C.byref(flags)))
    return int(flags.value)


def logistic_loss(pos: torch.Tensor, neg: Optional[torch.Tensor]):
    """(loss (1,), dpos, dneg): sum softplus(-pos) + mean-over-negatives-per-positive softplus(neg), and derivatives."""
    _need_cuda(pos, neg)
    dpos = torch.empty_like(pos)
    dneg = None if neg is None else torch.empty_like(neg)
    n_pos = pos.numel()
    n_neg = 0 if neg is None else neg.numel()
    w = 1.0 if n_neg == 0 else float(n_pos) / float(n_neg)
    loss = torch.empty(1, dtype=torch.float32, device=pos.device)
    ws = workspace(4096, pos.device, "loss")
    check(_lib.lib().kge_logistic_loss(_ptr(pos), n_pos, _ptr(neg), n_neg, w, _ptr(dpos), _ptr(dneg), _ptr(loss),
                                       _ptr(ws), ws.numel(), _stream()))
    return loss, dpos, dneg


# ---- scorers ----------------------------------------------------------------------------------------------
@dataclass
class SlotGrads:
    """Per-slot gradient rows of one backward call.  `ent_slots` is laid out like the id list [h | t | neg]."""
    ent_slots: torch.Tensor            # (2B + n_neg_ids, dim) fp32
    rel_slots: Optional[torch.Tensor]  # (B, dim) fp32: gradient of rel[r_i] per triple (None for RESCAL)
    rel2_slots: Optional[torch.Tensor]   # TransH: (B, dim) per triple
    rel2_groups: Optional[torch.Tensor]  # TransR/RESCAL: (n_groups_bound, dim, dim), group g <-> rel_insp.uniq[g]
    rel_insp: Optional[Inspection]       # grouping of the batch by relation (matrix models)


class Scorer:
    """A score function bound to its tables.

    model      "TransE" | "TransH" | "TransR" | "TransF" | "DistMult" | "RESCAL" | "ComplEx"
    ent        (n_ent, dim) float32 / bfloat16 entity table (ComplEx: interleaved re, im)
    rel        (n_rel, dim) relation vectors (None for RESCAL)
    rel2       TransH normals (n_rel, dim) or TransR/RESCAL matrices (n_rel, dim, dim)
    neg_mode   "none" | "per_triple" | "chunk_shared"; n_neg_head: leading negatives that replace the head
    """

    def __init__(self, model: str, ent: torch.Tensor, rel: Optional[torch.Tensor] = None,
                 rel2: Optional[torch.Tensor] = None, neg_mode: str = "none", n_neg_head: int = 0, chunk: int = 0,
                 precision: str = "fp32", check_ids: bool = False):
        if model not in MODELS:
            raise KeyError(model)
        self.precision = PRECISIONS[precision]
        self.flags = _lib.FLAG_CHECK_IDS if check_ids else 0     # ids are range-checked inside every scoring call
        _need_cuda(ent, rel, rel2)
        self.model, self.ent, self.rel, self.rel2 = model, ent, rel, rel2
        self.neg_mode, self.n_neg_head, self.chunk = neg_mode, int(n_neg_head), int(chunk)
        self.dim = ent.shape[1]
        self.n_rel = int((rel if rel is not None else rel2).shape[0])

    def with_entities(self, ent: torch.Tensor) -> "Scorer":
        """Same scorer over another entity buffer (e.g. the compact staging buffer of distinct rows)."""
        sc = Scorer(self.model, ent, self.rel, self.rel2, self.neg_mode, self.n_neg_head, self.chunk)
        sc.precision, sc.flags = self.precision, self.flags
        return sc

    # -- struct plumbing
    def _problem(self, h, neg) -> KgeProblem:
        n_neg = 0 if (neg is None or self.neg_mode == "none") else int(neg.shape[-1])
        return KgeProblem(MODELS[self.model], DTYPES[_dtype_of(self.ent)], NEG_MODES[self.neg_mode if n_neg else "none"],
                          _id_bits(h), self.dim, n_neg, self.n_neg_head if n_neg else 0,
                          self.chunk if self.neg_mode == "chunk_shared" else 0, h.numel(), self.ent.shape[0], self.n_rel,
                          self.precision, self.flags)

    def _tensors(self, h, r, t, neg, rel_insp: Optional[Inspection]) -> KgeTensors:
        kt = KgeTensors(_ptr(self.ent), _ptr(self.rel), _ptr(self.rel2), _ptr(h), _ptr(r), _ptr(t), _ptr(neg),
                        None, None, None, None)
        if rel_insp is not None:
            kt.rel_perm, kt.rel_seg = _ptr(rel_insp.perm), _ptr(rel_insp.seg)
            kt.rel_uniq, kt.n_rel_groups = _ptr(rel_insp.uniq), _ptr(rel_insp.n_unique)
        return kt

    def _check_ids(self, h, r, t, neg):
        _need_cuda(h, r, t, neg)
        bits = _id_bits(h)
        for x in (r, t, neg):
            if x is not None and _id_bits(x) != bits:
                raise TypeError("h, r, t, neg must share one integer dtype")
        if neg is not None and self.neg_mode == "per_triple" and neg.shape[0] != h.shape[0]:
            raise ValueError("per_triple negatives must be (batch, n_neg)")
        if neg is not None and self.neg_mode == "chunk_shared" and neg.shape[0] * self.chunk != h.shape[0]:
            raise ValueError("chunk_shared negatives must be (batch / chunk, n_neg)")

    def _group_by_relation(self, r) -> Inspection:
        """Inspector over the relation ids; with check_ids the grouping is built from the range-checked ids, because the
        relation-matrix kernels address P[rel_uniq[g]] through it."""
        if self.flags:
            checked = torch.empty_like(r)
            validate_ids(r, self.n_rel, checked)
            r = checked
        return inspect(r, self.n_rel)

    # -- reference-compatible output (what cuke's module.run returns)
    def ref_forward(self, h, r, t) -> torch.Tensor:
        self._check_ids(h, r, t, None)
        B = h.numel()
        out = torch.empty((B, self.dim) if self.model in VECTOR_MODELS else (B,), dtype=torch.float32, device=self.ent.device)
        p = self._problem(h, None)
        p.reserved = 0
        kt = self._tensors(h, r, t, None, None)
        check(_lib.lib().kge_ref_forward(C.byref(p), C.byref(kt), _ptr(out), _stream()))
        return out

    # -- scores
    def forward(self, h, r, t, neg=None, rel_insp: Optional[Inspection] = None):
        """(pos (B,), neg (B, n_neg) | (B/chunk, chunk, n_neg) | None, rel_insp)."""
        self._check_ids(h, r, t, neg)
        B = h.numel()
        dev = self.ent.device
        p = self._problem(h, neg)
        if self.model in MATRIX_MODELS and rel_insp is None:
            rel_insp = self._group_by_relation(r)
        kt = self._tensors(h, r, t, neg, rel_insp)
        pos = torch.empty(B, dtype=torch.float32, device=dev)
        negs = None
        if p.n_neg:
            shape = (B, p.n_neg) if self.neg_mode == "per_triple" else (B // self.chunk, self.chunk, p.n_neg)
            negs = torch.empty(shape, dtype=torch.float32, device=dev)
        L = _lib.lib()
        ws = workspace(L.kge_score_workspace_bytes(C.byref(p), 0), dev, "score")
        check(L.kge_score_forward(C.byref(p), C.byref(kt), _ptr(pos), _ptr(negs), _ptr(ws), ws.numel(), _stream()))
        return pos, negs, rel_insp

    def backward(self, h, r, t, neg, pos, negs, dpos, dneg, rel_insp: Optional[Inspection] = None,
                 ent_slots: Optional[torch.Tensor] = None) -> SlotGrads:
        self._check_ids(h, r, t, neg)
        _need_cuda(pos, negs, dpos, dneg)
        B, d, dev = h.numel(), self.dim, self.ent.device
        p = self._problem(h, neg)
        if self.model in MATRIX_MODELS and rel_insp is None:
            rel_insp = self._group_by_relation(r)
        kt = self._tensors(h, r, t, neg, rel_insp)
        n_neg_ids = neg.numel() if p.n_neg else 0
        n_slots = 2 * B + n_neg_ids
        if ent_slots is None:
            ent_slots = torch.empty((n_slots, d), dtype=torch.float32, device=dev)
        elif ent_slots.shape != (n_slots, d):
            raise ValueError("ent_slots has the wrong shape")
        rel_slots = rel2_slots = rel2_groups = None
        if self.model != "RESCAL":
            rel_slots = torch.empty((B, d), dtype=torch.float32, device=dev)
        if self.model == "TransH":
            rel2_slots = torch.empty((B, d), dtype=torch.float32, device=dev)
        if self.model in MATRIX_MODELS:
            rel2_groups = torch.zeros((min(self.n_rel, B), d, d), dtype=torch.float32, device=dev)
        g = KgeGrads(_ptr(ent_slots[:B]), _ptr(ent_slots[B:2 * B]), _ptr(ent_slots[2 * B:]) if n_neg_ids else None,
                     _ptr(rel_slots), _ptr(rel2_slots if rel2_slots is not None else rel2_groups))
        L = _lib.lib()
        ws = workspace(L.kge_score_workspace_bytes(C.byref(p), 1), dev, "score")
        check(L.kge_score_backward(C.byref(p), C.byref(kt), _ptr(pos), _ptr(negs), _ptr(dpos), _ptr(dneg), C.byref(g),
                                   _ptr(ws), ws.numel(), _stream()))
        return SlotGrads(ent_slots, rel_slots, rel2_slots, rel2_groups, rel_insp)


    def supports_fused_step(self, n_neg: int) -> bool:
        """True where loss_backward applies: tensor precision and either chunk-shared negatives with TransE / DistMult /
        ComplEx, or TransR over bf16 tables with per-triple negatives."""
        if self.precision == PRECISIONS["fp32"]:
            return False
        if self.model == "TransR":
            return (self.ent.dtype == torch.bfloat16 and self.dim % 8 == 0 and self.dim <= 256 and self.neg_mode != "chunk_shared")
        return (self.neg_mode == "chunk_shared" and self.dim % 4 == 0 and n_neg > 0 and self.model in ("TransE", "DistMult", "ComplEx"))

    def loss_backward(self, h, r, t, neg, neg_weight: Optional[float] = None,
                      ent_slots: Optional[torch.Tensor] = None, rel_insp: Optional[Inspection] = None):
        """forward -> logistic_loss -> backward in one call (kge_score_loss_backward): returns (pos, loss, SlotGrads).
        The scores of the negatives are consumed inside the call and are not returned."""
        self._check_ids(h, r, t, neg)
        B, d, dev = h.numel(), self.dim, self.ent.device
        p = self._problem(h, neg)
        rel2_groups = None
        if self.model in MATRIX_MODELS:
            if rel_insp is None:
                rel_insp = self._group_by_relation(r)
            rel2_groups = torch.zeros((min(self.n_rel, B), d, d), dtype=torch.float32, device=dev)
        kt = self._tensors(h, r, t, neg, rel_insp)
        if neg_weight is None:
            neg_weight = 1.0 / max(p.n_neg, 1)
        n_slots = 2 * B + (neg.numel() if p.n_neg else 0)
        if ent_slots is None:
            ent_slots = torch.empty((n_slots, d), dtype=torch.float32, device=dev)
        elif ent_slots.shape != (n_slots, d):
            raise ValueError("ent_slots has the wrong shape")
        rel_slots = torch.empty((B, d), dtype=torch.float32, device=dev)
        pos = torch.empty(B, dtype=torch.float32, device=dev)
        loss = torch.empty(1, dtype=torch.float32, device=dev)
        g = KgeGrads(_ptr(ent_slots[:B]), _ptr(ent_slots[B:2 * B]), _ptr(ent_slots[2 * B:]) if p.n_neg else None, _ptr(rel_slots),
                     _ptr(rel2_groups))
        L = _lib.lib()
        ws = workspace(L.kge_score_loss_backward_workspace_bytes(C.byref(p)), dev, "score")
        check(L.kge_score_loss_backward(C.byref(p), C.byref(kt), float(neg_weight), _ptr(pos), _ptr(loss), C.byref(g),
                                        _ptr(ws), ws.numel(), _stream()))
        return pos, loss, SlotGrads(ent_slots, rel_slots, None, rel2_groups, rel_insp)


def entity_id_list(h, t, neg) -> torch.Tensor:
    """The id list [h | t | neg] whose slots SlotGrads.ent_slots follows."""
    parts = [h.reshape(-1), t.reshape(-1)]
    if neg is not None:
        parts.append(neg.reshape(-1))
    return torch.cat(parts)
