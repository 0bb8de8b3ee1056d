"""Filter vocabularies as flat CSR arrays.

The reference keeps three pickled ``defaultdict(list)`` objects keyed by int tuples
(``er_vocab``: (h, r) → tails, ``re_vocab``: (r, t) → heads, ``ee_vocab``: (h, t) → relations;
reference ``dicee/static_funcs.py:75-126``).  Here the same information lives in three
sorted integer arrays (pair keys, offsets, values) that can be moved to the GPU as they
are and consumed by the label-construction and filtered-ranking kernels.  ``to_dict``
exports the reference's dictionary form so that the pickles on disk keep their layout.
"""
from __future__ import annotations

from collections import defaultdict
from typing import Dict, List, Tuple

import numpy as np
import torch


class PairCSR:
    """Mapping ``(a, b) -> sorted unique values`` stored as CSR over sorted pair keys.

    ``key = a * num_b + b``.  ``keys`` is strictly increasing, ``offsets`` has
    ``len(keys) + 1`` entries and ``values[offsets[i]:offsets[i+1]]`` are the values of
    pair ``i`` in ascending order.
    """

    def __init__(self, keys: np.ndarray, offsets: np.ndarray, values: np.ndarray, num_b: int):
        self.keys = keys.astype(np.int64, copy=False)
        self.offsets = offsets.astype(np.int64, copy=False)
        self.values = values.astype(np.int64, copy=False)
        self.num_b = int(num_b)
        self._torch_cache: Dict[str, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}

    # ------------------------------------------------------------------ construction
    @staticmethod
    def build(a: np.ndarray, b: np.ndarray, v: np.ndarray, num_b: int) -> "PairCSR":
        a = np.asarray(a, dtype=np.int64)
        b = np.asarray(b, dtype=np.int64)
        v = np.asarray(v, dtype=np.int64)
        if a.size == 0:
            return PairCSR(np.zeros(0, np.int64), np.zeros(1, np.int64), np.zeros(0, np.int64), num_b)
        key = a * int(num_b) + b
        order = np.lexsort((v, key))
        key, v = key[order], v[order]
        # drop duplicate (key, value) rows
        keep = np.ones(key.shape[0], dtype=bool)
        keep[1:] = (key[1:] != key[:-1]) | (v[1:] != v[:-1])
        key, v = key[keep], v[keep]
        uniq, start = np.unique(key, return_index=True)
        offsets = np.concatenate([start, [key.shape[0]]])
        return PairCSR(uniq, offsets, v, num_b)

    # ------------------------------------------------------------------ queries
    def __len__(self) -> int:
        return int(self.keys.shape[0])

    @property
    def pairs(self) -> np.ndarray:
        """``[num_pairs, 2]`` array of (a, b) in key order (lexicographic)."""
        return np.stack([self.keys // self.num_b, self.keys % self.num_b], axis=1)

    def counts(self) -> np.ndarray:
        return np.diff(self.offsets)

    def lookup(self, a: int, b: int) -> np.ndarray:
        k = int(a) * self.num_b + int(b)
        i = int(np.searchsorted(self.keys, k))
        if i >= len(self) or self.keys[i] != k:
            return self.values[:0]
        return self.values[self.offsets[i]:self.offsets[i + 1]]

    def to_dict(self) -> Dict[Tuple[int, int], List[int]]:
        out: Dict[Tuple[int, int], List[int]] = defaultdict(list)
        pairs = self.pairs
        off = self.offsets
        vals = self.values.tolist()
        for i, (x, y) in enumerate(pairs.tolist()):
            out[(x, y)] = vals[off[i]:off[i + 1]]
        return out

    def tensors(self, device="cpu") -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(keys, offsets, values) as int64 tensors on ``device`` (cached per device)."""
        dev = str(device)
        if dev not in self._torch_cache:
            self._torch_cache[dev] = (torch.from_numpy(self.keys).to(device),
                                      torch.from_numpy(self.offsets).to(device),
                                      torch.from_numpy(self.values).to(device))
        return self._torch_cache[dev]

    def batch_slices(self, a: torch.Tensor, b: torch.Tensor):
        """For query tensors ``a, b`` return ``(start, count)`` of each pair's value slice
        (count 0 for unseen pairs).  Runs on the device the queries live on."""
        keys, offsets, _ = self.tensors(a.device)
        k = a.long() * self.num_b + b.long()
        if keys.numel() == 0:
            z = torch.zeros_like(k)
            return z, z
        pos = torch.searchsorted(keys, k).clamp_(max=keys.numel() - 1)
        hit = keys[pos] == k
        start = offsets[pos]
        count = torch.where(hit, offsets[pos + 1] - start, torch.zeros_like(start))
        return start, count

    def batch_rows_cols(self, a: torch.Tensor, b: torch.Tensor):
        """Flattened (row, value) coordinates of all known values of the given pairs."""
        _, _, values = self.tensors(a.device)
        start, count = self.batch_slices(a, b)
        total = int(count.sum())
        rows = torch.repeat_interleave(torch.arange(a.shape[0], device=a.device), count)
        if total == 0:
            return rows, values[:0]
        first = torch.cumsum(count, 0) - count
        within = torch.arange(total, device=a.device) - torch.repeat_interleave(first, count)
        cols = values[torch.repeat_interleave(start, count) + within]
        return rows, cols


def er_csr(triples: np.ndarray, num_relations: int) -> PairCSR:
    return PairCSR.build(triples[:, 0], triples[:, 1], triples[:, 2], num_relations)


def re_csr(triples: np.ndarray, num_entities: int) -> PairCSR:
    return PairCSR.build(triples[:, 1], triples[:, 2], triples[:, 0], num_entities)


def ee_csr(triples: np.ndarray, num_entities: int) -> PairCSR:
    return PairCSR.build(triples[:, 0], triples[:, 2], triples[:, 1], num_entities)


from .vocab_writer import dict_vocab as _dict_vocab  # noqa: E402  (pure NumPy, shared with the helper process)


def get_er_vocab(data: np.ndarray) -> Dict[Tuple[int, int], List[int]]:
    """(head, relation) → list of tails in input order (reference ``static_funcs.py:75-90``)."""
    data = np.asarray(data)
    return _dict_vocab(data[:, 0], data[:, 1], data[:, 2])


def get_re_vocab(data: np.ndarray) -> Dict[Tuple[int, int], List[int]]:
    """(relation, tail) → list of heads (reference ``static_funcs.py:93-108``)."""
    data = np.asarray(data)
    return _dict_vocab(data[:, 1], data[:, 2], data[:, 0])


def get_ee_vocab(data: np.ndarray) -> Dict[Tuple[int, int], List[int]]:
    """(head, tail) → list of relations (reference ``static_funcs.py:111-126``)."""
    data = np.asarray(data)
    return _dict_vocab(data[:, 0], data[:, 2], data[:, 1])


def create_constraints(triples: np.ndarray):
    """Domain and range of every relation, and their complements.

    Returns ``(domain_constraints_per_rel, range_constraints_per_rel, domain_per_rel, range_per_rel)`` keyed by relation
    id: ``domain_per_rel[r]`` / ``range_per_rel[r]`` are the sets of entities seen as head / tail of ``r``; the
    ``*_constraints`` entries list the entities of the graph that were *never* seen there, i.e. the candidates a
    type-constrained ranking removes (reference ``dicee/static_preprocess_funcs.py:76-108``, which fills the same four
    dictionaries with one Python loop over the triples; here: one sort per side)."""
    assert isinstance(triples, np.ndarray) and triples.ndim == 2 and triples.shape[1] == 3
    t = triples.astype(np.int64, copy=False)
    entities = np.union1d(t[:, 0], t[:, 2])
    domain_per_rel, range_per_rel = {}, {}
    domain_constraints_per_rel, range_constraints_per_rel = {}, {}
    order = np.argsort(t[:, 1], kind="stable")
    rel_sorted = t[order, 1]
    rels, starts = np.unique(rel_sorted, return_index=True)
    ends = np.append(starts[1:], rel_sorted.shape[0])
    for r, a, b in zip(rels.tolist(), starts.tolist(), ends.tolist()):
        rows = order[a:b]
        dom, rng = np.unique(t[rows, 0]), np.unique(t[rows, 2])
        domain_per_rel[r], range_per_rel[r] = set(dom.tolist()), set(rng.tolist())
        domain_constraints_per_rel[r] = np.setdiff1d(entities, dom, assume_unique=True).tolist()
        range_constraints_per_rel[r] = np.setdiff1d(entities, rng, assume_unique=True).tolist()
    return domain_constraints_per_rel, range_constraints_per_rel, domain_per_rel, range_per_rel
