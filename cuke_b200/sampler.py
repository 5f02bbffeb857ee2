"""Batch ids generated on the GPU, and the triple-file format of the reference's datasets.

The reference draws every batch on the host: positives from a DGL EdgeSampler over the training graph, negatives per
chunk of `neg_sample_size` edges, flattened into ordinary triples and copied to the GPU
(apps/kge/data/data_init.py:19-63, apps/kge/data/sampler.py:287-353,395-504).  Here the ids are produced by kernels
of the library (kge_sample_uniform / kge_sample_cdf / kge_sample_triples: counter-based Philox, so a batch is a pure
function of (seed, step, rank)) straight into ONE buffer laid out [h | t | neg] - the id list the inspector sorts -
with `r` beside it; no host copy is involved.

`load_triples` reads the dataset layout the reference's preprocessing expects (apps/kge/data/preprocess.py:26-98):
`entities.dict` and `relations.dict` with one "<id>\t<name>" pair per line, `train.txt` with one
"<head>\t<relation>\t<tail>" name triple per line.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import check


def zipf_table(n_items: int, s: float = 1.1, perm_seed: int = 0, base_seed: int = 20240501) -> Tuple[np.ndarray, np.ndarray]:
    """(cdf float64 (n_items,), perm int64 (n_items,)): bounded Zipf(s) over ranks 1..n_items, ranks mapped to ids
    through a seeded permutation - the same table cuke_b200.synth.zipf_ids draws from on the host."""
    w = np.arange(1, n_items + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    perm = np.random.Generator(np.random.PCG64(base_seed + 7919 + perm_seed)).permutation(n_items).astype(np.int64)
    return cdf, perm


class DeviceSampler:
    """Seeded id batches on the current CUDA device.

    n_ent, n_rel     id spaces
    batch            positives per step
    n_neg            negatives per triple (per_triple) or per chunk (chunk_shared)
    neg_mode         "per_triple" | "chunk_shared" (then batch % chunk == 0)
    ent_dist         "uniform" | "zipf" (bounded Zipf(zipf_s) through a seeded permutation)
    triples          optional (n, 3) int64 tensor of (h, r, t) id triples: positives are drawn from it instead of
                     independently per column
    Streams: 4 per step and rank (h, t / triples, r, neg), stream id = 4 * (step * 65536 + rank) + k.
    """

    def __init__(self, n_ent: int, n_rel: int, batch: int, n_neg: int, neg_mode: str = "chunk_shared", chunk: int = 0,
                 ent_dist: str = "uniform", zipf_s: float = 1.1, seed: int = 20240501, rank: int = 0, id_dtype=torch.int64,
                 triples: Optional[torch.Tensor] = None, perm_seed: int = 0, device=None):
        self.n_ent, self.n_rel, self.batch, self.n_neg = int(n_ent), int(n_rel), int(batch), int(n_neg)
        self.neg_mode, self.chunk, self.seed, self.rank = neg_mode, int(chunk), int(seed), int(rank)
        if neg_mode == "chunk_shared" and (chunk <= 0 or batch % chunk):
            raise ValueError("chunk_shared needs batch % chunk == 0")
        if neg_mode not in ("per_triple", "chunk_shared"):
            raise ValueError(neg_mode)
        self.dev = device or torch.device("cuda", torch.cuda.current_device())
        self.id_dtype = id_dtype
        self.bits = 64 if id_dtype == torch.int64 else 32
        self.neg_shape = (batch, n_neg) if neg_mode == "per_triple" else (batch // chunk, n_neg)
        self.n_neg_ids = self.neg_shape[0] * self.neg_shape[1]
        self.cdf = self.perm = None
        if ent_dist == "zipf":
            cdf, perm = zipf_table(n_ent, zipf_s, perm_seed)
            self.cdf, self.perm = torch.from_numpy(cdf).to(self.dev), torch.from_numpy(perm).to(self.dev)
        elif ent_dist != "uniform":
            raise ValueError(ent_dist)
        self.triples = None
        if triples is not None:
            if triples.dtype != torch.int64 or triples.dim() != 2 or triples.shape[1] != 3:
                raise ValueError("triples must be an (n, 3) int64 tensor")
            self.triples = triples.to(self.dev).contiguous()

    def stream_id(self, step: int, k: int) -> int:
        return (4 * (step * 65536 + self.rank) + k) & 0xFFFFFFFF

    def _entities(self, out: torch.Tensor, step: int, k: int) -> None:
        L, s = _lib.lib(), torch.cuda.current_stream().cuda_stream
        if self.cdf is None:
            check(L.kge_sample_uniform(out.data_ptr(), self.bits, out.numel(), self.n_ent, self.seed, self.stream_id(step, k), s))
        else:
            check(L.kge_sample_cdf(out.data_ptr(), self.bits, out.numel(), self.cdf.data_ptr(), self.perm.data_ptr(), self.n_ent,
                                   self.seed, self.stream_id(step, k), s))

    def draw(self, step: int):
        """(ids, h, r, t, neg): `ids` is the whole list [h | t | neg]; h, t, neg are views into it, r its own tensor."""
        B = self.batch
        ids = torch.empty(2 * B + self.n_neg_ids, dtype=self.id_dtype, device=self.dev)
        r = torch.empty(B, dtype=self.id_dtype, device=self.dev)
        h, t, neg = ids[:B], ids[B:2 * B], ids[2 * B:].view(self.neg_shape)
        L, s = _lib.lib(), torch.cuda.current_stream().cuda_stream
        if self.triples is not None:
            check(L.kge_sample_triples(h.data_ptr(), r.data_ptr(), t.data_ptr(), self.bits, B, self.triples.data_ptr(),
                                       self.triples.shape[0], self.seed, self.stream_id(step, 1), s))
        else:
            self._entities(h, step, 0)
            self._entities(t, step, 1)
            check(L.kge_sample_uniform(r.data_ptr(), self.bits, B, self.n_rel, self.seed, self.stream_id(step, 2), s))
        self._entities(ids[2 * B:], step, 3)
        return ids, h, r, t, neg


def load_triples(path: str, split: str = "train.txt"):
    """Reads `entities.dict`, `relations.dict` and `<split>` under `path`; returns (triples (n, 3) int64 numpy array of
    (head id, relation id, tail id), n_entities, n_relations)."""
    def read_dict(name):
        m = {}
        with open(os.path.join(path, name)) as f:
            for line in f:
                line = line.rstrip("\n")
                if not line:
                    continue
                i, key = line.split("\t")
                m[key] = int(i)
        return m
    ent, rel = read_dict("entities.dict"), read_dict("relations.dict")
    rows = []
    with open(os.path.join(path, split)) as f:
        for line in f:
            line = line.rstrip("\n")
            if not line:
                continue
            hh, rr, tt = line.split("\t")
            rows.append((ent[hh], rel[rr], ent[tt]))
    return np.asarray(rows, dtype=np.int64).reshape(-1, 3), len(ent), len(rel)
