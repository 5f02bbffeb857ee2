"""Seeded synthetic workloads with the shapes and value distributions of the five benchmark configurations.

The reference's scripts draw batches from FB15k / FB15k-237 / wn18 / biokg through a DGL sampler
(apps/kge/data/data_init.py:19-63); neither the datasets nor DGL are available offline, so only shapes and
distributions are reproduced here: no dataset item is.  Everything is generated with numpy PCG64 streams,
one per tensor, seed = BASE_SEED + 1000 * config + tensor_index, so any process regenerates identical inputs.

  tables   rows ~ N(0, 1/dim) i.e. sigma = 1/sqrt(dim); TransH normals unit-normalised; relation matrices
           ~ N(0, 1/dim); ComplEx rows interleaved (re, im).
  ids      uniform, or bounded Zipf(s = 1.1) over ranks 1..N by inverse CDF, ranks mapped through a seeded
           permutation so that hot rows are spread over the id space (a contiguous row partition stays balanced).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

BASE_SEED = 20240501


@dataclass
class Config:
    name: str
    cid: int
    model: str
    n_ent: int
    n_rel: int
    dim: int
    batch: int
    n_neg: int
    neg_mode: str            # "per_triple" | "chunk_shared"
    n_neg_head: int = 0
    chunk: int = 0
    dtype: str = "f32"       # "f32" | "bf16"
    ent_dist: str = "uniform"  # "uniform" | "zipf"
    backward: bool = True
    extra_models: tuple = ()   # further scorers run on the same batch

    def scaled(self, ent: float = 1.0, batch: float = 1.0) -> "Config":
        """A smaller instance with the same structure (for parity tests)."""
        c = Config(**self.__dict__)
        c.n_ent = max(64, int(self.n_ent * ent))
        c.batch = max(1, int(self.batch * batch))
        if c.neg_mode == "chunk_shared":
            c.batch = max(c.chunk, c.batch // c.chunk * c.chunk)
        return c


CONFIGS = {
    "c1": Config("c1", 1, "TransE", 15000, 1350, 128, 1024, 64, "per_triple", 0, backward=False),
    "c2": Config("c2", 2, "TransH", 40000, 1350, 200, 4096, 256, "per_triple", 128),
    "c3": Config("c3", 3, "TransR", 40000, 1350, 200, 8192, 128, "per_triple", 64, dtype="bf16", ent_dist="zipf"),
    "c4": Config("c4", 4, "RESCAL", 100000, 500, 256, 16384, 256, "chunk_shared", 0, 256, ent_dist="zipf",
                 extra_models=("ComplEx",)),
    # c4 over bf16 tables (same ids and values, tables rounded to bf16; accumulation stays fp32)
    "c4_bf16": Config("c4_bf16", 4, "RESCAL", 100000, 500, 256, 16384, 256, "chunk_shared", 0, 256, dtype="bf16", ent_dist="zipf",
                      extra_models=("ComplEx",)),
    "c5": Config("c5", 5, "TransE", 4000000, 1000, 400, 65536, 1024, "chunk_shared", 0, 1024, ent_dist="zipf",
                 extra_models=("DistMult",)),
}


def _rng(cid: int, tensor_index: int, rank: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(BASE_SEED + 1000 * cid + tensor_index + 100000 * rank))


_zipf_cache = {}


def zipf_ids(rng: np.random.Generator, n_items: int, size, s: float = 1.1, perm_seed: int = 0) -> np.ndarray:
    """Bounded Zipf over ranks 1..n_items (p_k ~ k^-s) by inverse CDF; rank -> id through a seeded permutation."""
    key = (n_items, s, perm_seed)
    if key not in _zipf_cache:
        w = np.arange(1, n_items + 1, dtype=np.float64) ** (-s)
        cdf = np.cumsum(w)
        cdf /= cdf[-1]
        perm = np.random.Generator(np.random.PCG64(BASE_SEED + 7919 + perm_seed)).permutation(n_items)
        _zipf_cache[key] = (cdf, perm)
    cdf, perm = _zipf_cache[key]
    u = rng.random(size)
    ranks = np.searchsorted(cdf, u, side="left")
    np.clip(ranks, 0, n_items - 1, out=ranks)
    return perm[ranks].astype(np.int64)


def row_floats(cfg: Config, model: Optional[str] = None) -> int:
    """Floats per entity row: cfg.dim, or 2 * cfg.dim for ComplEx (cfg.dim complex numbers, interleaved re, im)."""
    return cfg.dim * 2 if (model or cfg.model) == "ComplEx" else cfg.dim


def make_tables(cfg: Config, model: Optional[str] = None):
    """(ent, rel, rel2) float32 numpy arrays for `model` (default cfg.model); rel/rel2 may be None."""
    model = model or cfg.model
    d = row_floats(cfg, model)
    sigma = 1.0 / np.sqrt(d)
    ent = _rng(cfg.cid, 1).standard_normal((cfg.n_ent, d), dtype=np.float32) * np.float32(sigma)
    rel = rel2 = None
    if model != "RESCAL":
        rel = _rng(cfg.cid, 2).standard_normal((cfg.n_rel, d), dtype=np.float32) * np.float32(sigma)
    if model == "TransH":
        w = _rng(cfg.cid, 3).standard_normal((cfg.n_rel, d), dtype=np.float32)
        rel2 = (w / np.linalg.norm(w, axis=1, keepdims=True)).astype(np.float32)
    if model in ("TransR", "RESCAL"):
        rel2 = _rng(cfg.cid, 4).standard_normal((cfg.n_rel, d, d), dtype=np.float32) * np.float32(sigma)
    return ent, rel, rel2


def make_batch(cfg: Config, step: int = 0, rank: int = 0):
    """(h, r, t, neg) int64 numpy arrays for one step of one rank."""
    base = 10 + 4 * step

    def ent_ids(ti, size):
        g = _rng(cfg.cid, base + ti, rank)
        if cfg.ent_dist == "zipf":
            return zipf_ids(g, cfg.n_ent, size, perm_seed=cfg.cid)
        return g.integers(0, cfg.n_ent, size=size, dtype=np.int64)

    h = ent_ids(0, cfg.batch)
    t = ent_ids(1, cfg.batch)
    r = _rng(cfg.cid, base + 2, rank).integers(0, cfg.n_rel, size=cfg.batch, dtype=np.int64)
    if cfg.neg_mode == "per_triple":
        neg = ent_ids(3, (cfg.batch, cfg.n_neg))
    else:
        neg = ent_ids(3, (cfg.batch // cfg.chunk, cfg.n_neg))
    return h, r, t, neg


def scored_triples(cfg: Config) -> int:
    """Positives + negatives scored per step (per scorer)."""
    if cfg.neg_mode == "per_triple":
        return cfg.batch * (1 + cfg.n_neg)
    return cfg.batch + (cfg.batch // cfg.chunk) * cfg.chunk * cfg.n_neg
