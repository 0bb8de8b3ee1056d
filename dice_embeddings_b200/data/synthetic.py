"""Seeded synthetic knowledge graphs.

The benchmark configurations name graph *shapes* (entity / relation / triple counts and a
degree distribution) rather than datasets, because no dataset can be downloaded on the
benchmark machines.  ``uniform_kg`` draws head, relation and tail uniformly;
``zipf_kg`` draws entity ids from a Zipf law over a random permutation of the entities
and relations from a second Zipf law.  Both remove duplicate triples and are pure
functions of their seed.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import numpy as np


def _zipf_sampler(n: int, s: float, rng: np.random.Generator):
    """Return ``draw(k)`` sampling ids in ``[0, n)`` with P(rank i) ∝ (i+1)^-s, ranks
    assigned to ids through a random permutation."""
    w = 1.0 / np.power(np.arange(1, n + 1, dtype=np.float64), s)
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    perm = rng.permutation(n)

    def draw(k: int) -> np.ndarray:
        u = rng.random(k)
        return perm[np.minimum(np.searchsorted(cdf, u), n - 1)]

    return draw


def _dedupe(tr: np.ndarray) -> np.ndarray:
    _, idx = np.unique(tr, axis=0, return_index=True)
    return tr[np.sort(idx)]


def uniform_kg(num_entities: int, num_relations: int, num_triples: int, seed: int = 0) -> np.ndarray:
    """``num_triples`` distinct (h, r, t) rows with every slot uniform at random."""
    rng = np.random.default_rng(seed)
    out = np.zeros((0, 3), dtype=np.int64)
    while out.shape[0] < num_triples:
        need = int((num_triples - out.shape[0]) * 1.2) + 16
        cand = np.stack([rng.integers(0, num_entities, need), rng.integers(0, num_relations, need),
                         rng.integers(0, num_entities, need)], axis=1)
        out = _dedupe(np.concatenate([out, cand]))
    return out[:num_triples]


def zipf_kg(num_entities: int, num_relations: int, num_triples: int, s_entity: float = 1.1,
            s_relation: float = 1.3, seed: int = 0) -> np.ndarray:
    """Distinct triples with Zipf-distributed heads/tails (over a random permutation) and relations; a first
    ``num_entities / 2`` triples pair up all entities so that the vocabulary has exactly ``num_entities`` entries."""
    rng = np.random.default_rng(seed)
    draw_e = _zipf_sampler(num_entities, s_entity, rng)
    draw_r = _zipf_sampler(num_relations, s_relation, rng)
    # coverage: every entity occurs at least once (pairs of a random permutation), the rest is Zipf
    cover = rng.permutation(num_entities)
    if cover.shape[0] % 2:
        cover = np.concatenate([cover, cover[:1]])
    out = np.stack([cover[0::2], draw_r(cover.shape[0] // 2), cover[1::2]], axis=1)[:num_triples]
    rounds = 0
    while out.shape[0] < num_triples and rounds < 64:
        need = int((num_triples - out.shape[0]) * 1.5) + 16
        cand = np.stack([draw_e(need), draw_r(need), draw_e(need)], axis=1)
        out = _dedupe(np.concatenate([out, cand]))
        rounds += 1
    return out[:num_triples]


def split_triples(triples: np.ndarray, num_valid: int, num_test: int, seed: int = 0
                  ) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Random split; every entity/relation of valid/test is guaranteed to occur in train by
    moving offending rows back (keeps the vocabulary identical across splits)."""
    rng = np.random.default_rng(seed + 7919)
    perm = rng.permutation(triples.shape[0])
    tr = triples[perm]
    hold = tr[: num_valid + num_test]
    train = tr[num_valid + num_test:]
    seen_e = np.zeros(int(triples[:, [0, 2]].max()) + 1, dtype=bool)
    seen_r = np.zeros(int(triples[:, 1].max()) + 1, dtype=bool)
    seen_e[train[:, 0]] = True
    seen_e[train[:, 2]] = True
    seen_r[train[:, 1]] = True
    ok = seen_e[hold[:, 0]] & seen_e[hold[:, 2]] & seen_r[hold[:, 1]]
    train = np.concatenate([train, hold[~ok]])
    hold = hold[ok]
    nv = min(num_valid, hold.shape[0] // 2 if num_test else hold.shape[0])
    return train, hold[:nv], hold[nv:nv + num_test]


def write_kg_folder(path: str, train: np.ndarray, valid: Optional[np.ndarray] = None,
                    test: Optional[np.ndarray] = None, entity_prefix: str = "e", relation_prefix: str = "r") -> str:
    """Write ``train.txt`` / ``valid.txt`` / ``test.txt`` with whitespace-separated string triples."""
    os.makedirs(path, exist_ok=True)

    def dump(name, arr):
        if arr is None or len(arr) == 0:
            return
        with open(os.path.join(path, name), "w") as f:
            f.write("\n".join(f"{entity_prefix}{h}\t{relation_prefix}{r}\t{entity_prefix}{t}"
                              for h, r, t in arr.tolist()))
            f.write("\n")

    dump("train.txt", train)
    dump("valid.txt", valid)
    dump("test.txt", test)
    return path


def make_umls_like(path: str, seed: int = 0) -> str:
    """135 entities, 46 relations, 5 216 / 652 / 661 triples drawn uniformly (benchmark config 1)."""
    tr = uniform_kg(135, 46, 5216 + 652 + 661, seed)
    train, valid, test = split_triples(tr, 652, 661, seed)
    return write_kg_folder(path, train, valid, test)


def make_fb15k237_like(path: str, seed: int = 0, with_eval_splits: bool = False) -> str:
    """14 541 entities, 237 relations, 272 115 train triples, Zipf(1.1) entities / Zipf(1.3) relations
    (benchmark config 2)."""
    extra = 17535 + 20466 if with_eval_splits else 0
    tr = zipf_kg(14541, 237, 272115 + extra, 1.1, 1.3, seed)
    if with_eval_splits:
        train, valid, test = split_triples(tr, 17535, 20466, seed)
        return write_kg_folder(path, train, valid, test)
    return write_kg_folder(path, tr)


def planted_kg(num_entities: int, num_relations: int, tails_per_pair: int = 3, pairs_per_relation: int = 60,
               dim: int = 8, seed: int = 0) -> np.ndarray:
    """Learnable synthetic graph: triples are the top-scoring tails of a hidden DistMult model, so a trained model
    can reach high filtered MRR on held-out triples (unlike uniformly random triples)."""
    rng = np.random.default_rng(seed)
    E = rng.normal(size=(num_entities, dim))
    R = rng.normal(size=(num_relations, dim))
    rows = []
    for r in range(num_relations):
        heads = rng.choice(num_entities, size=min(pairs_per_relation, num_entities), replace=False)
        scores = (E[heads] * R[r]) @ E.T
        top = np.argsort(-scores, axis=1)[:, :tails_per_pair]
        for h, ts in zip(heads, top):
            rows.extend((int(h), r, int(t)) for t in ts)
    return _dedupe(np.array(rows, dtype=np.int64))


def make_planted_kg(path: str, num_entities: int = 120, num_relations: int = 12, seed: int = 0) -> str:
    tr = planted_kg(num_entities, num_relations, seed=seed)
    n_hold = max(len(tr) // 10, 2)
    train, valid, test = split_triples(tr, n_hold, n_hold, seed)
    return write_kg_folder(path, train, valid, test)
