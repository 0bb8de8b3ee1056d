"""Out-of-core ingestion: triple files larger than memory → memory-mapped id triples → per-owner label CSR.

``index_triple_file`` streams a text file of ``s p o`` lines through the native indexer (``csrc/host/ingest.cpp``,
compiled with ``g++`` into ``libdice_ingest.so`` next to this file; a chunked pandas pass stands in where no compiler
is present) and leaves a run folder in the layout the executor and :class:`~dice_embeddings_b200.kge.KGE` read:

* ``memory_map_train_set.npy``  raw ``[n, 3]`` int32 array (opened with ``np.memmap``),
* ``memory_map_details.json``   ``{"shape": [n, 3], "dtype": "int32", "num_entities": …, "num_relations": …}``,
* ``entity_to_idx.csv`` / ``relation_to_idx.csv``  the vocabularies, ids in alphabetical order of the strings.

Only the vocabularies are ever held in memory.  ``owner_csr`` then builds, chunk by chunk from the memory map, the
``(head, relation) → known tails`` CSR restricted to the tails one rank of a row-sharded table owns, which is what
the label kernels of the sharded engines walk; ``MemmapTriples`` draws training batches straight from the map for the
sampled scoring techniques.

The reference does the same job in ``examples/train_kge_on_kg_larger_than_memory.py:17-63`` with polars joins over
batches, CSV chunks and a concatenated memory map.
"""
from __future__ import annotations

import ctypes
import json
import os
import subprocess
from typing import Dict, Iterator, Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(os.path.dirname(_HERE))
_SRC = os.path.join(_ROOT, "csrc", "host", "ingest.cpp")
LIB_PATH = os.path.join(_HERE, "libdice_ingest.so")
_lib: Optional[ctypes.CDLL] = None


def build(force: bool = False) -> str:
    """Compile the native indexer (host code only: ``g++ -O3 -shared``); no-op when the library is up to date."""
    if not force and os.path.isfile(LIB_PATH) and (not os.path.isfile(_SRC)
                                                    or os.path.getmtime(LIB_PATH) >= os.path.getmtime(_SRC)):
        return LIB_PATH
    tmp = f"{LIB_PATH}.{os.getpid()}.tmp"
    res = subprocess.run(["g++", "-O3", "-std=c++17", "-shared", "-fPIC", _SRC, "-o", tmp], capture_output=True,
                         text=True)
    if res.returncode != 0:
        raise RuntimeError(f"g++ failed on {_SRC}:\n{res.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


def native() -> Optional[ctypes.CDLL]:
    """The native indexer, or ``None`` when it cannot be built on this machine."""
    global _lib
    if _lib is None:
        try:
            build()
            _lib = ctypes.CDLL(LIB_PATH)
            _lib.dice_ingest_index_file.restype = ctypes.c_int
            _lib.dice_ingest_index_file.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p,
                                                    ctypes.c_int, ctypes.c_longlong,
                                                    ctypes.POINTER(ctypes.c_longlong)]
        except (RuntimeError, OSError, FileNotFoundError):
            _lib = None
    return _lib


def _index_with_pandas(path: str, triples_path: str, ent_path: str, rel_path: str, reciprocal: bool,
                       max_rows: Optional[int], chunk_rows: int) -> Tuple[int, int, int]:
    """Same result as the native indexer with two chunked pandas passes (vocabularies, then ids)."""
    import pandas as pd

    def chunks():
        seen = 0
        for df in pd.read_csv(path, sep=r"\s+", header=None, usecols=[0, 1, 2], names=["s", "p", "o"], dtype=str,
                              chunksize=chunk_rows, engine="python"):
            if max_rows is not None and seen + len(df) > max_rows:
                df = df.iloc[: max_rows - seen]
            seen += len(df)
            if len(df):
                yield df
            if max_rows is not None and seen >= max_rows:
                return

    ents, rels = set(), set()
    for df in chunks():
        ents.update(df["s"].tolist())
        ents.update(df["o"].tolist())
        rels.update(df["p"].tolist())
    if reciprocal:
        rels |= {r + "_inverse" for r in rels}
    ent_sorted, rel_sorted = sorted(ents), sorted(rels)
    e2i = {e: i for i, e in enumerate(ent_sorted)}
    r2i = {r: i for i, r in enumerate(rel_sorted)}
    n = 0
    with open(triples_path, "wb") as out:
        for df in chunks():
            s = df["s"].map(e2i).to_numpy(np.int32)
            p = df["p"].map(r2i).to_numpy(np.int32)
            o = df["o"].map(e2i).to_numpy(np.int32)
            if reciprocal:
                pi = (df["p"] + "_inverse").map(r2i).to_numpy(np.int32)
                block = np.empty((2 * len(df), 3), dtype=np.int32)
                block[0::2] = np.stack([s, p, o], 1)
                block[1::2] = np.stack([o, pi, s], 1)
            else:
                block = np.stack([s, p, o], 1)
            block.tofile(out)
            n += block.shape[0]
    for pth, items in ((ent_path, ent_sorted), (rel_path, rel_sorted)):
        with open(pth, "w") as f:
            f.write("\n".join(items) + ("\n" if items else ""))
    return n, len(ent_sorted), len(rel_sorted)


def index_triple_file(path: str, out_dir: str, reciprocal: bool = False, max_rows: Optional[int] = None,
                      use_native: Optional[bool] = None, chunk_rows: int = 2_000_000) -> Dict:
    """Index ``path`` into ``out_dir`` (see the module docstring for the files) and return the details dictionary."""
    os.makedirs(out_dir, exist_ok=True)
    triples_path = os.path.join(out_dir, "memory_map_train_set.npy")
    ent_list, rel_list = os.path.join(out_dir, "entities.txt"), os.path.join(out_dir, "relations.txt")
    lib = native() if use_native in (None, True) else None
    if use_native is True and lib is None:
        raise RuntimeError("the native indexer could not be built (g++ missing?)")
    if lib is not None:
        counts = (ctypes.c_longlong * 3)()
        rc = lib.dice_ingest_index_file(path.encode(), triples_path.encode(), ent_list.encode(), rel_list.encode(),
                                        int(reciprocal), int(max_rows or 0), counts)
        if rc != 0:
            why = {-1: "the input file cannot be opened", -2: "an output file cannot be written",
                   -3: "a line has fewer than three columns", -4: "too many distinct strings for 32-bit ids"}
            raise RuntimeError(f"indexing {path} failed: {why.get(rc, rc)}")
        n, ne, nr = int(counts[0]), int(counts[1]), int(counts[2])
        backend = "native"
    else:
        n, ne, nr = _index_with_pandas(path, triples_path, ent_list, rel_list, reciprocal, max_rows, chunk_rows)
        backend = "pandas"
    # vocabularies in the checkpoint layout (``pd.read_csv(index_col=0)`` reads them back)
    for src, dst, col in ((ent_list, "entity_to_idx.csv", "entity"), (rel_list, "relation_to_idx.csv", "relation")):
        with open(src) as f, open(os.path.join(out_dir, dst), "w") as g:
            g.write(f",{col}\n")
            for i, line in enumerate(f):
                item = line.rstrip("\n")
                if any(c in item for c in ',"\n'):
                    item = '"' + item.replace('"', '""') + '"'
                g.write(f"{i},{item}\n")
    details = {"shape": [n, 3], "dtype": "int32", "num_entities": ne, "num_relations": nr, "indexer": backend}
    with open(os.path.join(out_dir, "memory_map_details.json"), "w") as f:
        json.dump(details, f, indent=4)
    return details


def open_triples(run_dir: str) -> np.memmap:
    """Read-only memory map of the triples indexed into ``run_dir``."""
    with open(os.path.join(run_dir, "memory_map_details.json")) as f:
        d = json.load(f)
    return np.memmap(os.path.join(run_dir, "memory_map_train_set.npy"), mode="r", dtype=d["dtype"],
                     shape=tuple(d["shape"]))


def owner_csr(triples: np.ndarray, num_relations: int, world: int = 1, rank: int = 0,
              chunk_rows: int = 20_000_000) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """``(pairs [P, 2], offsets [P + 1], values)``: the distinct ``(head, relation)`` pairs of ``triples`` in sorted
    order and, for each, the known tails *owned by* ``rank`` (``tail % world == rank``) as local row numbers
    (``tail // world``).  ``triples`` may be a memory map: it is read in chunks of ``chunk_rows`` rows and only keys
    and the owned tails are kept, i.e. every rank of a sharded run holds ``1 / world`` of the label store."""
    keys, tails = [], []
    n = triples.shape[0]
    for a in range(0, n, chunk_rows):
        blk = np.asarray(triples[a:a + chunk_rows])
        key = blk[:, 0].astype(np.int64) * num_relations + blk[:, 1].astype(np.int64)
        keys.append(np.unique(key))                        # every pair is a data point, owned tails or not
        own = (blk[:, 2] % world) == rank
        tails.append((key[own], (blk[own, 2] // world).astype(np.int64)))
    all_keys = np.unique(np.concatenate(keys)) if keys else np.zeros(0, dtype=np.int64)
    tk = np.concatenate([t[0] for t in tails]) if tails else np.zeros(0, dtype=np.int64)
    tv = np.concatenate([t[1] for t in tails]) if tails else np.zeros(0, dtype=np.int64)
    order = np.lexsort((tv, tk))
    tk, tv = tk[order], tv[order]
    if tk.size:                                            # duplicate triples contribute one label
        keep = np.ones(tk.size, dtype=bool)
        keep[1:] = (tk[1:] != tk[:-1]) | (tv[1:] != tv[:-1])
        tk, tv = tk[keep], tv[keep]
    counts = np.zeros(all_keys.size + 1, dtype=np.int64)
    np.add.at(counts, np.searchsorted(all_keys, tk) + 1, 1)
    offsets = np.cumsum(counts)
    pairs = np.stack([all_keys // num_relations, all_keys % num_relations], axis=1)
    return pairs, offsets, tv


class MemmapTriples:
    """Batches of training triples drawn straight from a memory map (sampled scoring techniques: the negatives are
    drawn on the device by the engines, so a batch is just ``B`` rows of the map)."""

    def __init__(self, triples: np.ndarray, batch_size: int, seed: int = 0):
        self.triples, self.batch_size = triples, int(batch_size)
        self.rng = np.random.default_rng(seed)

    def __len__(self) -> int:
        return -(-self.triples.shape[0] // self.batch_size)

    def __iter__(self) -> Iterator:
        import torch
        n = self.triples.shape[0]
        # random contiguous windows: page-friendly on a map that does not fit in memory
        starts = self.rng.permutation(len(self)) * self.batch_size
        for s in starts:
            blk = np.asarray(self.triples[s:min(s + self.batch_size, n)])
            if blk.shape[0] < self.batch_size:
                blk = np.concatenate([blk, np.asarray(self.triples[: self.batch_size - blk.shape[0]])])
            yield torch.from_numpy(blk.astype(np.int64))
