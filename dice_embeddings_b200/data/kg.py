"""Knowledge-graph container: read → (reciprocals, noise) → sorted vocabulary → int triples → disk.

Behaviour follows the reference pipeline (``dicee/knowledge_graph.py:114-122``:
``ReadFromDisk`` → ``PreprocessKG`` → ``LoadSaveToDisk``), re-implemented as one class
working on NumPy string arrays:

* files named ``*train*``, ``*valid*``, ``*test*`` of a folder, a single KG file, or a SPARQL
  endpoint (reference ``read_from_disk.py:13-61``); valid/test are only read when
  ``eval_model`` is set;
* reciprocal triples ``(t, r_inverse, h)`` are appended to every split when
  ``add_reciprocal and eval_model`` (reference ``util.py:126-131``);
* entity and relation vocabularies are the **alphabetically sorted** unique strings
  (reference ``preprocess.py:382-384``), so ids are a pure function of the data;
* triples are stored with the smallest integer dtype that fits (reference
  ``static_funcs.py:373-392``);
* ``entity_to_idx.csv`` / ``relation_to_idx.csv`` use the pandas layout (unnamed index column +
  ``entity`` / ``relation`` column), ``{train,valid,test}_set.npy`` hold the index triples
  (reference ``save_load_disk.py:34-44``).

The three filter vocabularies are built as CSR arrays (:mod:`.vocab`) and exported as the
reference's pickled dictionaries on demand.
"""
from __future__ import annotations

import glob
import atexit
import os
import pickle
import sys
from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np
import pandas as pd

from .bpe import get_tokenizer
from .vocab import PairCSR, ee_csr, er_csr, get_ee_vocab, get_er_vocab, get_re_vocab, re_csr


def shrink_int_dtype(arr: np.ndarray, num: int) -> np.ndarray:
    """Smallest signed integer dtype able to hold ``num`` (reference ``static_funcs.py:373-392``)."""
    for dt in (np.int8, np.int16, np.int32):
        if np.iinfo(dt).max > num:
            return arr.astype(dt)
    return arr.astype(np.int64)


# ----------------------------------------------------------------------------- readers
def _read_table(path: str, read_only_few=None, sample_triples_ratio=None, backend="pandas",
                separator=r"\s+") -> pd.DataFrame:
    ext = os.path.splitext(path)[1].lower().lstrip(".")
    if ext in ("ttl", "owl", "turtle", "rdf/xml", "rdf") and backend != "rdflib":
        raise RuntimeError(f"Data with **{ext}** format cannot be read via --backend pandas or polars. "
                           f"Use --backend rdflib")
    if backend == "rdflib":
        try:
            from rdflib import Graph
        except ModuleNotFoundError as e:  # optional dependency
            raise ModuleNotFoundError("--backend rdflib needs the rdflib package") from e
        df = pd.DataFrame([(str(s), str(p), str(o)) for s, p, o in Graph().parse(path)],
                          columns=["subject", "relation", "object"], dtype=str)
    elif backend == "polars":
        try:
            import polars
            sep = "\t" if separator in (r"\s+", "t", "\\t") else separator
            df = polars.read_csv(path, has_header=False, n_rows=read_only_few, columns=[0, 1, 2],
                                 new_columns=["subject", "relation", "object"], separator=sep,
                                 infer_schema_length=0).to_pandas()
        except (ImportError, AttributeError, RuntimeError) as exc:
            # polars is optional (absent, or a stub that refuses to read); pandas reads the same files
            print(f"--backend polars is not usable here ({type(exc).__name__}); reading {path} with pandas instead")
            df = pd.read_csv(path, sep=separator, header=None, nrows=read_only_few, usecols=[0, 1, 2],
                             names=["subject", "relation", "object"], dtype=str)
    elif ext in ("nt", "ttl", "txt", "csv", "zst", "tsv"):
        df = pd.read_csv(path, sep=separator, header=None, nrows=read_only_few, usecols=[0, 1, 2],
                         names=["subject", "relation", "object"], dtype=str)
    else:
        df = pd.read_parquet(path, engine="pyarrow")
        df.columns = ["subject", "relation", "object"][: len(df.columns)]
        if read_only_few and read_only_few > 0:
            df = df.head(read_only_few)
    if sample_triples_ratio:
        df = df.sample(frac=sample_triples_ratio)
    # RDF n-triples: drop rows whose object is a literal (reference util.py:149-158)
    head = df.head()
    if (head["subject"].str.startswith("<").sum() + head["relation"].str.startswith("<").sum()) > 2:
        df = df[df["object"].str.startswith("<", na=False)]
    return df.reset_index(drop=True)


_SPARQL_HEADERS = {"Content-Type": "application/x-www-form-urlencoded", "Accept": "application/sparql-results+json"}


def count_triples(endpoint: str) -> int:
    """Total number of triples in the store behind ``endpoint`` (reference ``util.py:244-258``)."""
    import requests
    resp = requests.post(endpoint, data={"query": "SELECT (COUNT(*) AS ?count) WHERE { ?s ?p ?o . }"},
                         headers=_SPARQL_HEADERS)
    resp.raise_for_status()
    return int(resp.json()["results"]["bindings"][0]["count"]["value"])


def _fetch_page(endpoint: str, offset: int, chunk_size: int) -> pd.DataFrame:
    import requests
    query = f"SELECT ?subject ?predicate ?object WHERE {{ ?subject ?predicate ?object . }} LIMIT {chunk_size} OFFSET {offset}"
    resp = requests.post(endpoint, data={"query": query}, headers=_SPARQL_HEADERS)
    if not resp.ok:   # the reference skips a failed page with a message; so does this reader
        print(f"SPARQL page at offset {offset} failed: {getattr(resp, 'status_code', '?')}")
        return pd.DataFrame(columns=["subject", "relation", "object"], dtype=str)
    rows = [(b["subject"]["value"], b["predicate"]["value"], b["object"]["value"])
            for b in resp.json()["results"]["bindings"]]
    return pd.DataFrame(rows, columns=["subject", "relation", "object"], dtype=str)


def _read_sparql(endpoint: str, chunk_size: int = 500_000, num_workers: Optional[int] = None,
                 cache_dir: Optional[str] = None) -> pd.DataFrame:
    """All (s, p, o) of a triple store, fetched in pages of ``chunk_size`` rows with ``LIMIT / OFFSET`` queries that
    run concurrently (a thread per page in flight: the work is waiting for the endpoint), in offset order.

    The reference counts the triples, deals the page offsets to one worker *process* per core, parks every page as a
    parquet file and re-reads the folder (``dicee/read_preprocess_save_load_kg/util.py:244-328``).  ``cache_dir`` keeps
    that behaviour: pages are written there as ``chunk_<offset>.parquet`` and an existing folder is read back instead
    of querying again."""
    from concurrent.futures import ThreadPoolExecutor
    if cache_dir and os.path.isdir(cache_dir):
        files = sorted(glob.glob(os.path.join(cache_dir, "chunk_*.parquet")),
                       key=lambda f: int(os.path.basename(f)[6:-8]))
        if files:
            print(f"*** Found parquet files in `{cache_dir}`, reading from those; delete the folder to query again ***")
            return pd.concat([pd.read_parquet(f) for f in files], ignore_index=True).astype(str)
    total = count_triples(endpoint)
    offsets = list(range(0, total, chunk_size))
    workers = max(1, min(num_workers or (os.cpu_count() or 1), len(offsets) or 1))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        pages = list(pool.map(lambda off: _fetch_page(endpoint, off, chunk_size), offsets))
    if cache_dir:
        os.makedirs(cache_dir, exist_ok=True)
        for off, page in zip(offsets, pages):
            if len(page):
                page.to_parquet(os.path.join(cache_dir, f"chunk_{off}.parquet"), index=False)
    pages = [pg for pg in pages if len(pg)]
    if not pages:
        return pd.DataFrame(columns=["subject", "relation", "object"], dtype=str)
    return pd.concat(pages, ignore_index=True)


def add_reciprocals(df: Optional[pd.DataFrame]) -> Optional[pd.DataFrame]:
    if df is None:
        return None
    inv = pd.DataFrame({"subject": df["object"].values,
                        "relation": df["relation"].astype(str).values + "_inverse",
                        "object": df["subject"].values})
    return pd.concat([df, inv], ignore_index=True)


def add_noisy_triples(df: pd.DataFrame, rate: float, seed: int = 0) -> pd.DataFrame:
    """Append ``rate · len(df)`` random triples over the seen entities / relations
    (reference ``read_from_disk.py:63-78``)."""
    n = int(len(df) * rate)
    if n <= 0:
        return df
    rng = np.random.default_rng(seed)
    ents = pd.unique(df[["subject", "object"]].values.ravel("K"))
    rels = pd.unique(df["relation"].values)
    noise = pd.DataFrame({"subject": rng.choice(ents, n), "relation": rng.choice(rels, n),
                          "object": rng.choice(ents, n)})
    return pd.concat([df, noise], ignore_index=True)


# ----------------------------------------------------------------------------- container
class KG:
    """Indexed knowledge graph with train / valid / test splits."""

    def __init__(self, dataset_dir: Optional[str] = None, byte_pair_encoding: bool = False, padding: bool = False,
                 add_noise_rate: Optional[float] = None, sparql_endpoint: Optional[str] = None,
                 path_single_kg: Optional[str] = None, path_for_deserialization: Optional[str] = None,
                 add_reciprocal: Optional[bool] = None, eval_model: Optional[str] = None,
                 read_only_few: Optional[int] = None, sample_triples_ratio: Optional[float] = None,
                 path_for_serialization: Optional[str] = None, entity_to_idx: Optional[Dict] = None,
                 relation_to_idx: Optional[Dict] = None, backend: Optional[str] = None,
                 training_technique: Optional[str] = None, separator: Optional[str] = None):
        self.dataset_dir = dataset_dir
        self.sparql_endpoint = sparql_endpoint
        self.path_single_kg = path_single_kg
        self.byte_pair_encoding = byte_pair_encoding
        self.padding = padding
        self.add_noise_rate = add_noise_rate
        self.path_for_deserialization = path_for_deserialization
        self.add_reciprocal = add_reciprocal
        self.eval_model = eval_model
        self.read_only_few = read_only_few
        self.sample_triples_ratio = sample_triples_ratio
        self.path_for_serialization = path_for_serialization
        self.entity_to_idx = entity_to_idx
        self.relation_to_idx = relation_to_idx
        self.backend = backend or "pandas"
        self.training_technique = training_technique
        self.separator = separator or r"\s+"
        self.num_entities: Optional[int] = None
        self.num_relations: Optional[int] = None
        self.raw_train_set = self.raw_valid_set = self.raw_test_set = None
        self.train_set = self.valid_set = self.test_set = None
        self.er_vocab = self.re_vocab = self.ee_vocab = None
        self._er_csr = self._re_csr = self._ee_csr = None
        self.domain_constraints_per_rel = self.range_constraints_per_rel = None
        # byte-pair-encoding state
        self.enc = get_tokenizer() if byte_pair_encoding else None
        self.num_tokens = self.enc.n_vocab if self.enc is not None else None
        self.dummy_id = self.enc.encode(" ")[0] if self.enc is not None else None
        self.max_length_subword_tokens: Optional[int] = None
        self.ordered_bpe_entities = None
        self.ordered_bpe_relations = None
        self.train_target_indices = None
        self.target_dim: Optional[int] = None
        self.num_bpe_entities: Optional[int] = None

        if path_for_deserialization is None:
            self._read()
            if byte_pair_encoding:
                self._preprocess_bpe()
            else:
                self._preprocess()
            self._build_filter_vocab()
            self.save()
        else:
            self.load()
        assert len(self.train_set) > 0, "Training set is empty"
        self.description_of_input = None
        self.describe()
        if isinstance(self.entity_to_idx, dict):
            self.idx_to_entity = {v: k for k, v in self.entity_to_idx.items()}
            self.idx_to_relations = {v: k for k, v in self.relation_to_idx.items()}

    # ------------------------------------------------------------------ reading
    def _read(self) -> None:
        kw = dict(backend=self.backend, separator=self.separator)
        if self.path_single_kg is not None:
            self.raw_train_set = _read_table(self.path_single_kg, self.read_only_few, self.sample_triples_ratio, **kw)
        elif self.sparql_endpoint is not None:
            self.raw_train_set = _read_sparql(self.sparql_endpoint)
        elif self.dataset_dir:
            for f in sorted(glob.glob(self.dataset_dir + "/*")):
                name = os.path.basename(f)
                if "train" in name:
                    self.raw_train_set = _read_table(f, self.read_only_few, self.sample_triples_ratio, **kw)
                elif "test" in name and self.eval_model is not None:
                    self.raw_test_set = _read_table(f, **kw)
                elif "valid" in name and self.eval_model is not None:
                    self.raw_valid_set = _read_table(f, **kw)
            if self.raw_train_set is None:
                raise RuntimeError(f"No file containing 'train' found under {self.dataset_dir}")
        else:
            raise RuntimeError(f"Invalid data: {self.dataset_dir}\t{self.sparql_endpoint}\t{self.path_single_kg}")
        if self.add_noise_rate:
            self.raw_train_set = add_noisy_triples(self.raw_train_set, self.add_noise_rate)

    def _apply_reciprocals(self) -> None:
        if self.add_reciprocal and self.eval_model:
            self.raw_train_set = add_reciprocals(self.raw_train_set)
            self.raw_valid_set = add_reciprocals(self.raw_valid_set)
            self.raw_test_set = add_reciprocals(self.raw_test_set)

    # ------------------------------------------------------------------ indexing
    def _preprocess(self) -> None:
        self._apply_reciprocals()
        splits = [s for s in (self.raw_train_set, self.raw_valid_set, self.raw_test_set) if s is not None]
        ents = np.concatenate([np.concatenate([s["subject"].values, s["object"].values]) for s in splits]).astype(str)
        rels = np.concatenate([s["relation"].values for s in splits]).astype(str)
        if self.entity_to_idx is None:
            # pandas sort_values on object strings == Python string order == np.unique on a str array
            ent_sorted = sorted(set(ents.tolist()))
            rel_sorted = sorted(set(rels.tolist()))
            self.entity_to_idx = {e: i for i, e in enumerate(ent_sorted)}
            self.relation_to_idx = {r: i for i, r in enumerate(rel_sorted)}
        self.num_entities, self.num_relations = len(self.entity_to_idx), len(self.relation_to_idx)
        max_idx = max(self.num_entities, self.num_relations)

        def index(df):
            if df is None:
                return None
            h = df["subject"].astype(str).map(self.entity_to_idx).values
            r = df["relation"].astype(str).map(self.relation_to_idx).values
            t = df["object"].astype(str).map(self.entity_to_idx).values
            arr = np.stack([h, r, t], axis=1).astype(np.int64)
            assert arr.shape[0] > 0, "Size of the dataset must be greater than 0."
            return shrink_int_dtype(arr, max_idx)

        self.train_set = index(self.raw_train_set)
        self.valid_set = index(self.raw_valid_set)
        self.test_set = index(self.raw_test_set)
        from ..config import dataset_sanity_checking
        dataset_sanity_checking(self.train_set, self.num_entities, self.num_relations)

    def _preprocess_bpe(self) -> None:
        """Token-id triples, optionally padded to a common length
        (reference ``preprocess.py:186-256`` and ``:62-121``)."""
        self._apply_reciprocals()
        enc = self.enc

        def encode(df):
            if df is None:
                return []
            return [tuple(tuple(enc.encode(str(x))) for x in row) for row in df.itertuples(index=False, name=None)]

        train, valid, test = encode(self.raw_train_set), encode(self.raw_valid_set), encode(self.raw_test_set)
        if not self.padding:
            space, end = enc.encode(" ")[0], enc.encode(".")[0]
            stream: List[int] = []
            for h, r, t in train:
                stream.extend([*h, space, *r, space, *t, end])
            self.train_set = np.array(stream)
            self.valid_set = valid or None
            self.test_set = test or None
            return
        self.max_length_subword_tokens = max(max(len(h), len(r), len(t)) for h, r, t in train + valid + test)
        T = self.max_length_subword_tokens
        ent_shaped: Dict[tuple, tuple] = {}
        rel_shaped: Dict[tuple, tuple] = {}

        def pad(x):
            return x + (self.dummy_id,) * (T - len(x))

        def shape(rows):
            out = []
            for s, p, o in rows:
                se, pe, oe = pad(s), pad(p), pad(o)
                ent_shaped[s], ent_shaped[o], rel_shaped[p] = se, oe, pe
                out.append((se, pe, oe))
            return out

        train, valid, test = shape(train), shape(valid), shape(test)
        self.ordered_bpe_entities = sorted([(enc.decode(k), k, v) for k, v in ent_shaped.items()], key=lambda x: x[0])
        self.ordered_bpe_relations = sorted([(enc.decode(k), k, v) for k, v in rel_shaped.items()], key=lambda x: x[0])
        self.num_bpe_entities = len(self.ordered_bpe_entities)
        self.bpe_valid_set = valid
        self.bpe_test_set = test
        self.bpe_train_triples = train
        if self.training_technique in ("KvsAll", "AllvsAll"):
            ent_idx = {shaped: i for i, (_, _, shaped) in enumerate(self.ordered_bpe_entities)}
            er_tails: Dict[tuple, list] = {}
            for h, r, t in train:
                er_tails.setdefault((h, r), []).append(ent_idx[t])
            if self.training_technique == "AllvsAll":
                toks = {s for (_, _, s) in self.ordered_bpe_entities + self.ordered_bpe_relations}
                for i in toks:
                    for j in toks:
                        er_tails.setdefault((i, j), [])
            self.train_set = np.array([list(k) for k in er_tails.keys()])
            self.train_target_indices = list(er_tails.values())
            self.target_dim = len(self.ordered_bpe_entities)
        else:  # NegSample keeps padded token triples [N, 3, T]
            self.train_set = np.array(train)
        self.valid_set = np.array(valid) if valid else None
        self.test_set = np.array(test) if test else None

    def _build_filter_vocab(self) -> None:
        if not self.eval_model or self.byte_pair_encoding:
            if self.eval_model and self.byte_pair_encoding and self.padding:
                data = [tuple(x) for x in (self.bpe_train_triples + self.bpe_valid_set + self.bpe_test_set)]
                er, re_, ee = {}, {}, {}
                for h, r, t in data:
                    er.setdefault((h, r), []).append(t)
                    re_.setdefault((r, t), []).append(h)
                    ee.setdefault((h, t), []).append(r)
                self.er_vocab, self.re_vocab, self.ee_vocab = er, re_, ee
            return
        # reference preprocess.py:51-54: all three splits only when both valid and test exist
        if isinstance(self.valid_set, np.ndarray) and isinstance(self.test_set, np.ndarray):
            data = np.concatenate([self.train_set, self.valid_set, self.test_set]).astype(np.int64)
        else:
            data = self.train_set.astype(np.int64)
        self._filter_data = data
        self._er_csr = er_csr(data, self.num_relations)
        self._re_csr = re_csr(data, self.num_entities)
        self._ee_csr = None  # built lazily, rarely needed

    # CSR accessors -------------------------------------------------------------------
    @property
    def er_csr(self) -> PairCSR:
        return self._er_csr

    @property
    def re_csr(self) -> PairCSR:
        return self._re_csr

    @property
    def ee_csr(self) -> PairCSR:
        if self._ee_csr is None and getattr(self, "_filter_data", None) is not None:
            self._ee_csr = ee_csr(self._filter_data, self.num_entities)
        return self._ee_csr

    def materialize_dict_vocab(self) -> None:
        """Fill ``er_vocab`` / ``re_vocab`` / ``ee_vocab`` with the reference's dict-of-lists form."""
        if self.er_vocab is None and getattr(self, "_filter_data", None) is not None:
            self.er_vocab = get_er_vocab(self._filter_data)
            self.re_vocab = get_re_vocab(self._filter_data)
            self.ee_vocab = get_ee_vocab(self._filter_data)

    # ------------------------------------------------------------------ persistence
    def save(self) -> None:
        p = self.path_for_serialization
        if p is None:
            return
        os.makedirs(p, exist_ok=True)
        if self.byte_pair_encoding:
            np.save(os.path.join(p, "train_set.npy"), self.train_set)
            with open(os.path.join(p, "ordered_bpe_entities.p"), "wb") as f:
                pickle.dump(self.ordered_bpe_entities, f)
            with open(os.path.join(p, "ordered_bpe_relations.p"), "wb") as f:
                pickle.dump(self.ordered_bpe_relations, f)
            return
        pd.DataFrame({"entity": list(self.entity_to_idx.keys())}).to_csv(os.path.join(p, "entity_to_idx.csv"),
                                                                        header=True)
        pd.DataFrame({"relation": list(self.relation_to_idx.keys())}).to_csv(
            os.path.join(p, "relation_to_idx.csv"), header=True)
        np.save(os.path.join(p, "train_set.npy"), self.train_set)
        if self.valid_set is not None:
            np.save(os.path.join(p, "valid_set.npy"), self.valid_set)
        if self.test_set is not None:
            np.save(os.path.join(p, "test_set.npy"), self.test_set)

    def save_filter_vocab_pickles(self, path: Optional[str] = None, background: bool = False) -> None:
        """Write ``er_vocab.p`` / ``re_vocab.p`` / ``ee_vocab.p`` (reference ``preprocess.py:58-60``).

        ``background=True`` hands the job to a helper process (``data/vocab_writer.py`` run as a script on a copy of
        the filter triples) and returns at once; :meth:`wait_for_vocab_pickles` joins it.  Nothing in this framework
        reads the dictionaries while a run is in progress: filtering uses the CSR form."""
        path = path or self.path_for_serialization
        if path is None or not self.eval_model:
            return
        if background and self.er_vocab is None and getattr(self, "_filter_data", None) is not None:
            import subprocess
            import sys
            from . import vocab_writer
            tmp = os.path.join(path, f".filter_triples.{os.getpid()}.npy")
            np.save(tmp, np.asarray(self._filter_data))
            self._vocab_writer = subprocess.Popen([sys.executable, os.path.abspath(vocab_writer.__file__), tmp, path])
            atexit.register(self.wait_for_vocab_pickles)
            return
        self.materialize_dict_vocab()
        for name in ("er_vocab", "re_vocab", "ee_vocab"):
            obj = getattr(self, name)
            if obj is not None:
                with open(os.path.join(path, name + ".p"), "wb") as f:
                    pickle.dump(obj, f)

    def wait_for_vocab_pickles(self) -> None:
        """Join the helper process of :meth:`save_filter_vocab_pickles`; falls back to writing them here if it failed."""
        proc = getattr(self, "_vocab_writer", None)
        if proc is None:
            return
        self._vocab_writer = None
        if proc.wait() != 0:
            self.save_filter_vocab_pickles(proc.args[3])

    def load(self) -> None:
        p = self.path_for_deserialization
        ent = pd.read_csv(os.path.join(p, "entity_to_idx.csv"), index_col=0)
        rel = pd.read_csv(os.path.join(p, "relation_to_idx.csv"), index_col=0)
        self.entity_to_idx = {str(v): int(i) for i, v in zip(ent.index, ent.iloc[:, 0])}
        self.relation_to_idx = {str(v): int(i) for i, v in zip(rel.index, rel.iloc[:, 0])}
        self.num_entities, self.num_relations = len(self.entity_to_idx), len(self.relation_to_idx)
        self.train_set = np.load(os.path.join(p, "train_set.npy"))
        if os.path.isfile(os.path.join(p, "valid_set.npy")):
            self.valid_set = np.load(os.path.join(p, "valid_set.npy"))
        if os.path.isfile(os.path.join(p, "test_set.npy")):
            self.test_set = np.load(os.path.join(p, "test_set.npy"))
        self._build_filter_vocab()

    # ------------------------------------------------------------------ misc API
    def describe(self) -> None:
        source = self.dataset_dir or self.sparql_endpoint or self.path_single_kg or self.path_for_deserialization
        lines = [f'\n{"=" * 20} Description of Dataset {source} {"=" * 20}']
        if self.byte_pair_encoding:
            lines += [f"Number of tokens: {self.num_tokens}",
                      f"Max sequence length of sub-words: {self.max_length_subword_tokens}"]
        else:
            lines += [f"Number of entities: {self.num_entities}", f"Number of relations: {self.num_relations}"]
        lines += [f"Number of triples on train set: {len(self.train_set)}",
                  f"Number of triples on valid set: {len(self.valid_set) if self.valid_set is not None else 0}",
                  f"Number of triples on test set: {len(self.test_set) if self.test_set is not None else 0}"]
        if not self.byte_pair_encoding:
            lines += [f"Entity Index: {sys.getsizeof(self.entity_to_idx) / 1e9:.5f} GB",
                      f"Relation Index: {sys.getsizeof(self.relation_to_idx) / 1e9:.5f} GB"]
        self.description_of_input = "\n".join(lines)

    @property
    def entities_str(self) -> List[str]:
        return list(self.entity_to_idx.keys())

    @property
    def relations_str(self) -> List[str]:
        return list(self.relation_to_idx.keys())

    def exists(self, h: str, r: str, t: str) -> bool:
        """True when the string triple is in the training split."""
        try:
            row = (self.entity_to_idx[h], self.relation_to_idx[r], self.entity_to_idx[t])
        except KeyError:
            return False
        ts = self.train_set
        return bool(((ts[:, 0] == row[0]) & (ts[:, 1] == row[1]) & (ts[:, 2] == row[2])).any())

    def __iter__(self) -> Iterator[Tuple[str, str, str]]:
        for h, r, t in np.asarray(self.train_set).tolist():
            yield self.idx_to_entity[h], self.idx_to_relations[r], self.idx_to_entity[t]

    def __len__(self) -> int:
        return len(self.train_set)

    def func_triple_to_bpe_representation(self, triple: List[str]):
        """Token ids of (h, r, t), each padded to ``max_length_subword_tokens``
        (reference ``knowledge_graph.py:204-215``)."""
        out = []
        for x in triple:
            ids = list(self.enc.encode(x))
            ids += [self.dummy_id] * max(0, self.max_length_subword_tokens - len(ids))
            out.append(ids)
        return out
