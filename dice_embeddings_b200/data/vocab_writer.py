"""Dict-of-lists filter vocabularies (``er_vocab.p`` / ``re_vocab.p`` / ``ee_vocab.p``) of a run folder.

The framework itself filters with CSR arrays; the pickled dictionaries are kept in the run folder because the
reference writes them there (``dicee/evaluation/evaluator.py:66-78``) and existing tooling reads them.  Building them
is pure host work on Python objects, so the evaluator hands it to a helper process: this file run as a script (it
imports nothing but NumPy, so the helper starts in a fraction of a second) while the ranking runs on the device.  The
reference overlaps the same work with a process pool started when the graph is loaded
(``dicee/knowledge_graph.py:104-113``).

    python vocab_writer.py <triples.npy> <run folder>
"""
from __future__ import annotations

import gc
import os
import pickle
import sys
from collections import defaultdict
from typing import Dict, List, Tuple

import numpy as np


def dict_vocab(a, b, v) -> Dict[Tuple[int, int], List[int]]:
    """``(a, b) → [v, ...]`` in input order per key: one stable sort, then one list slice per distinct key.  The
    cyclic garbage collector is paused meanwhile: with it, allocating hundreds of thousands of small containers
    triggers full collections that triple the time."""
    out: Dict[Tuple[int, int], List[int]] = defaultdict(list)
    a, b, v = np.asarray(a, dtype=np.int64), np.asarray(b, dtype=np.int64), np.asarray(v)
    if a.size == 0:
        return out
    key = a * (int(b.max()) + 1) + b
    order = np.argsort(key, kind="stable")
    ks = key[order]
    starts = np.flatnonzero(np.concatenate([[True], ks[1:] != ks[:-1]]))
    ends = np.concatenate([starts[1:], [ks.size]])
    vals = v[order].tolist()
    ka, kb = a[order][starts].tolist(), b[order][starts].tolist()
    was_on = gc.isenabled()
    gc.disable()
    try:
        out.update({(x, y): vals[s:e] for x, y, s, e in zip(ka, kb, starts.tolist(), ends.tolist())})
    finally:
        if was_on:
            gc.enable()
    return out


def write_pickles(data: np.ndarray, folder: str) -> None:
    """The three vocabularies of ``data [n, 3]`` (head, relation, tail), each written to a temporary name first."""
    for name, (i, j, k) in (("er_vocab", (0, 1, 2)), ("re_vocab", (1, 2, 0)), ("ee_vocab", (0, 2, 1))):
        obj = dict_vocab(data[:, i], data[:, j], data[:, k])
        tmp = os.path.join(folder, f".{name}.{os.getpid()}.tmp")
        with open(tmp, "wb") as f:
            pickle.dump(obj, f, protocol=pickle.HIGHEST_PROTOCOL)
        os.replace(tmp, os.path.join(folder, name + ".p"))
        del obj


if __name__ == "__main__":
    write_pickles(np.load(sys.argv[1]), sys.argv[2])
    os.remove(sys.argv[1])
