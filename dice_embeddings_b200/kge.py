"""Interactive inference / fine-tuning API over a stored run: ``KGE(path=…)``.

Public surface of the reference class (``dicee/knowledge_graph_embeddings.py:10-1330`` plus the mix-ins in
``dicee/abstracts.py:153-871``): ``predict``, ``predict_topk``, ``triple_score``, the three
``predict_missing_*`` helpers, ``answer_multi_hop_query``, ``find_missing_triples``, ``train`` /
``train_triples`` / ``train_k_vs_all``, ``train_literals`` / ``predict_literals``, ``save`` and the embedding
accessors.  Implementation differences: candidate scoring is batched (one model call per chunk of queries
instead of one per query), multi-hop queries are evaluated by a small recursive interpreter over the query
structure with beam projection done in one batched call, and everything runs on the model's device.
"""
from __future__ import annotations

import datetime
import os
import random
import sys
from typing import Dict, Iterable, List, Optional, Set, Tuple, Union

import numpy as np
import pandas as pd
import torch
import torch.nn.functional as F

from .data.bpe import get_tokenizer
from .data.datasets import LiteralDataset, TriplePredictionDataset
from .evaluation.link_prediction import evaluate_lp
from .io.checkpoint import (load_json, load_model, load_model_ensemble, load_pickle, save_checkpoint_model)
from .models.literal import LiteralEmbeddings
from .trainer.base import BatchLoader

StrOrList = Union[List[str], str]

# EPFO + negation query structures and their short names (reference knowledge_graph_embeddings.py:700-716)
QUERY_NAME = {
    ("e", ("r",)): "1p",
    ("e", ("r", "r")): "2p",
    ("e", ("r", "r", "r")): "3p",
    (("e", ("r",)), ("e", ("r",))): "2i",
    (("e", ("r",)), ("e", ("r",)), ("e", ("r",))): "3i",
    ((("e", ("r",)), ("e", ("r",))), ("r",)): "ip",
    (("e", ("r", "r")), ("e", ("r",))): "pi",
    (("e", ("r",)), ("e", ("r", "n"))): "2in",
    (("e", ("r",)), ("e", ("r",)), ("e", ("r", "n"))): "3in",
    ((("e", ("r",)), ("e", ("r", "n"))), ("r",)): "inp",
    (("e", ("r", "r")), ("e", ("r", "n"))): "pin",
    (("e", ("r", "r", "n")), ("e", ("r",))): "pni",
    (("e", ("r",)), ("e", ("r",)), ("u",)): "2u",
    ((("e", ("r",)), ("e", ("r",)), ("u",)), ("r",)): "up",
}


def download_pretrained_model(url: str) -> str:
    """Mirror the files listed at ``url`` into a local folder named after its last path component
    (reference ``dicee/static_funcs.py:738-796``).  Needs network access."""
    import re
    import requests
    name = url.rstrip("/").split("/")[-1]
    dest = os.path.join(os.getcwd(), name)
    if os.path.isdir(dest) and os.listdir(dest):
        return dest
    os.makedirs(dest, exist_ok=True)
    page = requests.get(url, timeout=30)
    page.raise_for_status()
    for href in set(re.findall(r'href="([^"?/][^"]*)"', page.text)):
        if href.endswith("/"):
            continue
        r = requests.get(url.rstrip("/") + "/" + href, timeout=120)
        if r.ok:
            with open(os.path.join(dest, os.path.basename(href)), "wb") as f:
                f.write(r.content)
    return dest


class KGE:
    def __init__(self, path: str = None, url: str = None, construct_ensemble: bool = False, model_name: str = None,
                 apply_semantic_constraint: bool = False):
        if url is not None:
            assert path is None
            path = download_pretrained_model(url)
        self.path = path
        assert self.path is not None and os.path.isdir(self.path), f"Could not find a directory {self.path}"
        self.construct_ensemble = construct_ensemble
        self.apply_semantic_constraint = apply_semantic_constraint
        self.configs = load_json(os.path.join(self.path, "configuration.json"))
        if os.path.isfile(os.path.join(self.path, "report.json")):
            self.configs.update(load_json(os.path.join(self.path, "report.json")))
        if construct_ensemble:
            self.model, maps = load_model_ensemble(self.path)
        else:
            self.model, maps = load_model(self.path, model_name=model_name) if model_name else load_model(self.path)
        self.literal_model = None
        self.literal_dataset = None
        if self.configs.get("byte_pair_encoding", None):
            self.enc = get_tokenizer()
            self.dummy_id = self.enc.encode(" ")[0]
            self.max_length_subword_tokens = self.configs.get("max_length_subword_tokens")
            obe = self.configs.get("ordered_bpe_entities")
            if obe is None and os.path.isfile(os.path.join(self.path, "ordered_bpe_entities.p")):
                obe = load_pickle(os.path.join(self.path, "ordered_bpe_entities.p"))
            if obe:
                self.entity_to_idx = {s: i for i, (s, _, _) in enumerate(obe)}
                self.idx_to_entity = {i: s for s, i in self.entity_to_idx.items()}
                self.num_entities = len(self.entity_to_idx)
        else:
            self.entity_to_idx, self.relation_to_idx = maps
            self.num_entities, self.num_relations = len(self.entity_to_idx), len(self.relation_to_idx)
            assert sorted(self.entity_to_idx.values()) == list(range(self.num_entities))
            assert sorted(self.relation_to_idx.values()) == list(range(self.num_relations))
            self.idx_to_entity = {v: k for k, v in self.entity_to_idx.items()}
            self.idx_to_relations = {v: k for k, v in self.relation_to_idx.items()}
        self._train_set = None
        if hasattr(self, "relation_to_idx"):
            base = [r for r in self.relation_to_idx if not r.endswith("_inverse")]
            self.all_have_inverse = all(f"{r}_inverse" in self.relation_to_idx for r in base)
        else:
            self.all_have_inverse = False
        self._maybe_load_literal_model()

    # ------------------------------------------------------------------ basics
    def __str__(self):
        return "KGE | " + str(self.model)

    def to(self, device: str) -> None:
        assert "cpu" in device or "cuda" in device, "Device must be either cpu or cuda"
        self.model.to(device)

    @property
    def name(self):
        return self.model.name

    @property
    def train_set(self) -> np.ndarray:
        if self._train_set is None:
            self._train_set = np.load(os.path.join(self.path, "train_set.npy"))
        return self._train_set

    def get_eval_report(self) -> dict:
        return load_json(os.path.join(self.path, "eval_report.json"))

    def parameters(self):
        return self.model.parameters()

    def set_model_train_mode(self) -> None:
        self.model.train()
        for p in self.model.parameters():
            p.requires_grad = True

    def set_model_eval_mode(self) -> None:
        self.model.eval()
        for p in self.model.parameters():
            p.requires_grad = False

    def sample_entity(self, n: int) -> List[str]:
        return random.sample(list(self.entity_to_idx.keys()), n)

    def sample_relation(self, n: int) -> List[str]:
        return random.sample(list(self.relation_to_idx.keys()), n)

    def is_seen(self, entity: str = None, relation: str = None) -> bool:
        if entity is not None:
            return entity in self.entity_to_idx
        if relation is not None:
            return relation in self.relation_to_idx
        return False

    def save(self) -> None:
        t = str(datetime.datetime.now())
        tag = "model_ensemble_interactive_" if self.construct_ensemble else "model_interactive_"
        save_checkpoint_model(self.model, path=os.path.join(self.path, f"{tag}{t}.pt"))

    def get_entity_index(self, x: str) -> int:
        return self.entity_to_idx[x]

    def get_relation_index(self, x: str) -> int:
        return self.relation_to_idx[x]

    def index_triple(self, head_entity: List[str], relation: List[str], tail_entity: List[str]):
        n = len(head_entity)
        assert n == len(relation) == len(tail_entity)
        h = torch.LongTensor([self.entity_to_idx[i] for i in head_entity]).reshape(n, 1)
        r = torch.LongTensor([self.relation_to_idx[i] for i in relation]).reshape(n, 1)
        t = torch.LongTensor([self.entity_to_idx[i] for i in tail_entity]).reshape(n, 1)
        return h, r, t

    def construct_input_and_output(self, head_entity, relation, tail_entity, labels):
        h, r, t = self.index_triple(head_entity, relation, tail_entity)
        return torch.hstack((h, r, t)), torch.FloatTensor(labels)

    def add_new_entity_embeddings(self, entity_name: str = None, embeddings: torch.FloatTensor = None):
        assert isinstance(entity_name, str) and isinstance(embeddings, torch.Tensor)
        if entity_name in self.entity_to_idx:
            print(f"Entity ({entity_name}) exists..")
            return
        idx = len(self.entity_to_idx)
        self.entity_to_idx[entity_name] = idx
        self.idx_to_entity[idx] = entity_name
        self.num_entities += 1
        self.model.num_entities += 1
        w = self.model.entity_embeddings.weight.data
        self.model.entity_embeddings.weight.data = torch.cat((w.detach(), embeddings.to(w).reshape(1, -1)), dim=0)
        self.model.entity_embeddings.num_embeddings += 1

    def get_entity_embeddings(self, items: List[str]):
        if self.configs.get("byte_pair_encoding"):
            tok = [self.get_bpe_token_representation(i) for i in items]
            return self.model.token_embeddings(torch.LongTensor(tok).to(self.model.device)).flatten(1)
        idx = torch.LongTensor([self.entity_to_idx[i] for i in items]).to(self.model.device)
        return self.model.entity_embeddings(idx)

    def get_relation_embeddings(self, items: List[str]):
        idx = torch.LongTensor([self.relation_to_idx[i] for i in items]).to(self.model.device)
        return self.model.relation_embeddings(idx)

    def get_transductive_entity_embeddings(self, indices, as_pytorch=False, as_numpy=False, as_list=True):
        if not isinstance(indices, torch.Tensor):
            assert isinstance(indices, list)
            indices = torch.LongTensor([self.entity_to_idx[i] for i in indices])
        emb = self.model.entity_embeddings(indices.to(self.model.device)).detach()
        if as_pytorch:
            return emb
        if as_numpy:
            return emb.cpu().numpy()
        if as_list:
            return emb.tolist()
        raise RuntimeError("Something went wrong with the types")

    # byte-pair helpers ---------------------------------------------------------------
    def get_bpe_token_representation(self, x: StrOrList):
        if isinstance(x, list):
            return [self.get_bpe_token_representation(i) for i in x]
        # padded to the training-time width; longer strings are cut there (the reference leaves that case open,
        # ``dicee/abstracts.py:241-243``)
        ids = list(self.enc.encode(x))[: self.max_length_subword_tokens]
        ids += [self.dummy_id] * max(0, self.max_length_subword_tokens - len(ids))
        return ids

    def get_padded_bpe_triple_representation(self, triples: List[List[str]]):
        if not isinstance(triples[0], list):
            triples = [triples]
        hs, rs, ts = [], [], []
        for s, p, o in triples:
            hs.append(self.get_bpe_token_representation(s))
            rs.append(self.get_bpe_token_representation(p))
            ts.append(self.get_bpe_token_representation(o))
        return hs, rs, ts

    # ------------------------------------------------------------------ vector database
    def create_vector_database(self, collection_name: str, distance: str, location: str = "localhost",
                               port: int = 6333):
        """Push all entity embeddings into a Qdrant collection (needs the optional ``qdrant_client``)."""
        assert distance in ("cosine", "dot")
        try:
            from qdrant_client import QdrantClient
            from qdrant_client.http.models import Distance, PointStruct, VectorParams
        except ModuleNotFoundError as e:
            raise ModuleNotFoundError("Please install qdrant_client: pip install qdrant_client") from e
        client = QdrantClient(location=location, port=port)
        if collection_name in [c.name for c in client.get_collections().collections]:
            client.delete_collection(collection_name=collection_name)
        dist = Distance.COSINE if distance == "cosine" else Distance.DOT
        client.create_collection(collection_name=collection_name,
                                 vectors_config=VectorParams(size=self.model.embedding_dim, distance=dist))
        ents = list(self.idx_to_entity.values())
        vecs = self.get_transductive_entity_embeddings(indices=ents, as_list=True)
        pts = [PointStruct(id=self.entity_to_idx[e], vector=v, payload={"name": e}) for e, v in zip(ents, vecs)]
        return client.upsert(collection_name=collection_name, wait=True, points=pts)

    # ------------------------------------------------------------------ evaluation
    def eval_lp_performance(self, dataset: List[Tuple[str, str, str]] = None, filtered: bool = True):
        assert isinstance(dataset, list) and len(dataset) > 0
        idx = np.array([(self.entity_to_idx[s], self.relation_to_idx[p], self.entity_to_idx[o]) for s, p, o in dataset])
        if filtered:
            return evaluate_lp(self.model, idx, len(self.entity_to_idx),
                               load_pickle(os.path.join(self.path, "er_vocab.p")),
                               load_pickle(os.path.join(self.path, "re_vocab.p")))
        return evaluate_lp(self.model, idx, len(self.entity_to_idx), None, None)

    # ------------------------------------------------------------------ prediction helpers
    def _ent_ids(self, x: StrOrList) -> torch.Tensor:
        return torch.LongTensor([self.entity_to_idx[i] for i in (x if isinstance(x, list) else [x])])

    def _rel_ids(self, x: StrOrList) -> torch.Tensor:
        return torch.LongTensor([self.relation_to_idx[i] for i in (x if isinstance(x, list) else [x])])

    @torch.no_grad()
    def _collect(self, n_rows: int, width: int, batch_size: int, topk: int, return_indices: bool, score_rows):
        """Run ``score_rows(i, j) -> [j-i, width]`` over row chunks; gather flat scores or per-row top-k."""
        if return_indices:
            scores = torch.zeros(n_rows, topk)
            indices = torch.zeros(n_rows, topk, dtype=torch.long)
        else:
            scores = torch.zeros(n_rows * width)
        for i in range(0, n_rows, batch_size):
            j = min(i + batch_size, n_rows)
            s = score_rows(i, j)
            if return_indices:
                v, ix = torch.topk(s, topk, dim=1)
                scores[i:j], indices[i:j] = v.cpu(), ix.cpu()
            else:
                scores[i * width:j * width] = s.flatten().cpu()
        return (scores.flatten(), indices.flatten()) if return_indices else scores

    @torch.no_grad()
    def _fused_topk(self, pairs: torch.Tensor, topk: int, batch_size: int):
        """Top-k tails through the tcgen05 ranking kernel (no ``[B, |E|]`` score matrix); ``None`` when the model is
        outside what the kernel covers."""
        from .ops import eval_rank
        if not eval_rank.supports(self.model):
            return None
        ranker = eval_rank.ranker_for_model(self.model, exact=False)  # rebuilt per call: the weights may have been trained since
        dev = self.model.device
        scores, indices = [], []
        for i in range(0, pairs.shape[0], batch_size):
            q, bias = eval_rank.model_queries(self.model, pairs[i:i + batch_size].to(dev))
            s, ix = ranker.topk(q, topk)
            scores.append((s if bias is None else s + bias.reshape(-1, 1)).cpu())
            indices.append(ix.cpu())
        ranker.check()
        return torch.cat(scores).flatten(), torch.cat(indices).flatten()

    def predict_missing_head_entity(self, relation: StrOrList, tail_entity: StrOrList, within=None,
                                    batch_size: int = 2, topk: int = 1, return_indices: bool = False):
        """Scores of every entity as head for each ``(tail, relation)`` of the Cartesian product.  When every
        relation has an ``_inverse`` twin the query is rewritten as tail prediction with the inverse relation
        (reference ``knowledge_graph_embeddings.py:139-228``)."""
        if self.all_have_inverse:
            rel = [f"{r}_inverse" for r in (relation if isinstance(relation, list) else [relation])]
            return self.predict_missing_tail_entity(tail_entity, rel, within, batch_size, topk, return_indices)
        pairs = torch.cartesian_prod(self._ent_ids(tail_entity), self._rel_ids(relation))
        H = len(self.entity_to_idx)
        dev = self.model.device
        heads = torch.arange(H, device=dev)

        def rows(i, j):
            b = pairs[i:j].to(dev)
            B = b.shape[0]
            x = torch.stack((heads.repeat(B), b[:, 1].repeat_interleave(H), b[:, 0].repeat_interleave(H)), dim=1)
            return self.model(x).view(B, H)

        return self._collect(pairs.shape[0], H, batch_size, topk, return_indices, rows)

    def predict_missing_relations(self, head_entity: StrOrList, tail_entity: StrOrList, within=None,
                                  batch_size: int = 2, topk: int = 1, return_indices: bool = False):
        pairs = torch.cartesian_prod(self._ent_ids(head_entity), self._ent_ids(tail_entity))
        R = len(self.relation_to_idx)
        dev = self.model.device
        rels = torch.arange(R, device=dev)

        def rows(i, j):
            b = pairs[i:j].to(dev)
            B = b.shape[0]
            x = torch.stack((b[:, 0].repeat_interleave(R), rels.repeat(B), b[:, 1].repeat_interleave(R)), dim=1)
            return self.model(x).view(B, R)

        return self._collect(pairs.shape[0], R, batch_size, topk, return_indices, rows)

    def predict_missing_tail_entity(self, head_entity: StrOrList, relation: StrOrList, within: List[str] = None,
                                    batch_size: int = 2, topk: int = 1, return_indices: bool = False):
        if within is not None:  # byte-pair-encoded models: score only the given candidate strings
            h = head_entity[0] if isinstance(head_entity, list) else head_entity
            r = relation[0] if isinstance(relation, list) else relation
            n = len(within)
            ht = torch.LongTensor(self.get_bpe_token_representation(h)).unsqueeze(0).expand(n, -1)
            rt = torch.LongTensor(self.get_bpe_token_representation(r)).unsqueeze(0).expand(n, -1)
            tt = torch.LongTensor(self.get_bpe_token_representation(list(within)))
            with torch.no_grad():
                return self.model(torch.stack((ht, rt, tt), dim=1).to(self.model.device))
        pairs = torch.cartesian_prod(self._ent_ids(head_entity), self._rel_ids(relation))
        T = len(self.entity_to_idx)
        dev = self.model.device
        if return_indices and topk <= 32 and dev.type == "cuda":
            fused = self._fused_topk(pairs, topk, max(batch_size, 1024))
            if fused is not None:
                return fused
        return self._collect(pairs.shape[0], T, batch_size, topk, return_indices,
                             lambda i, j: self.model(pairs[i:j].to(dev)).view(j - i, T))

    def predict(self, *, h: StrOrList = None, r: StrOrList = None, t: StrOrList = None, within=None,
                logits: bool = True) -> torch.FloatTensor:
        """Scores for the missing slot (all candidates, flattened) or for a full triple."""
        for v in (h, r, t):
            if v is not None:
                assert isinstance(v, (list, str)) and isinstance(v[0], str)
        if h is None:
            assert r is not None and t is not None
            s = self.predict_missing_head_entity(r, t, within, batch_size=64, topk=len(self.entity_to_idx))
        elif r is None:
            assert t is not None
            s = self.predict_missing_relations(h, t, within, batch_size=64, topk=len(self.relation_to_idx))
        elif t is None:
            s = self.predict_missing_tail_entity(h, r, within, batch_size=64, topk=len(self.entity_to_idx))
        else:
            s = self.triple_score(h, r, t, logits=True)
        return s if logits else torch.sigmoid(s)

    def predict_topk(self, *, h: StrOrList = None, r: StrOrList = None, t: StrOrList = None, topk: int = 10,
                     within: List[str] = None, batch_size: int = 1024):
        """Top-``k`` completions with sigmoid scores: one list of ``(string, probability)`` per query pair."""
        as_list = lambda v: [v] if isinstance(v, str) else v  # noqa: E731
        if h is None:
            assert r is not None and t is not None
            r, t = as_list(r), as_list(t)
            fs, fi = self.predict_missing_head_entity(r, t, within, batch_size, topk, return_indices=True)
            n, lookup = len(r) * len(t), self.idx_to_entity
        elif r is None:
            assert t is not None
            h, t = as_list(h), as_list(t)
            fs, fi = self.predict_missing_relations(h, t, within, batch_size, topk, return_indices=True)
            n, lookup = len(h) * len(t), self.idx_to_relations
        elif t is None:
            h, r = as_list(h), as_list(r)
            fs, fi = self.predict_missing_tail_entity(h, r, within, batch_size, topk, return_indices=True)
            n, lookup = len(h) * len(r), self.idx_to_entity
        else:
            raise AttributeError("Use triple_score method")
        probs = torch.sigmoid(fs.view(n, topk)).tolist()
        idxs = fi.view(n, topk).tolist()
        return [[(lookup[i], s) for i, s in zip(ri, rs)] for ri, rs in zip(idxs, probs)]

    @torch.no_grad()
    def triple_score(self, h: StrOrList = None, r: StrOrList = None, t: StrOrList = None, logits: bool = False):
        if self.configs.get("byte_pair_encoding", None):
            rows = [self.get_bpe_token_representation(v) for v in (h, r, t)]
            x = torch.LongTensor(rows).unsqueeze(0)
        elif isinstance(h, list) and isinstance(r, list) and isinstance(t, list):
            x = torch.hstack(self.index_triple(h, r, t))
        else:
            x = torch.hstack(self.index_triple([h], [r], [t]))
        out = self.model(x.to(self.model.device))
        if self.apply_semantic_constraint:
            # a triple whose head lies outside the relation's domain or whose tail lies outside its range (as seen in
            # the training graph) cannot hold: logit -inf, probability 0.  The reference names the switch but raises
            # NotImplementedError here (dicee/knowledge_graph_embeddings.py:642-643).
            ok = self._semantic_mask(x)
            out = torch.where(ok.to(out.device), out, torch.full_like(out, float("-inf")))
        return out if logits else torch.sigmoid(out)

    def semantic_constraints(self):
        """``(domain_constraints_per_rel, range_constraints_per_rel, domain_per_rel, range_per_rel)`` of the stored
        training triples, computed once (reference ``dicee/static_preprocess_funcs.py:76-108``)."""
        if getattr(self, "_constraints", None) is None:
            from .data.vocab import create_constraints
            self._constraints = create_constraints(np.asarray(self.train_set))
        return self._constraints

    def _semantic_mask(self, x: torch.Tensor) -> torch.Tensor:
        _, _, dom, rng = self.semantic_constraints()
        rows = x.view(-1, 3).tolist()
        return torch.tensor([h in dom.get(r, ()) and t in rng.get(r, ()) for h, r, t in rows], dtype=torch.bool)

    # ------------------------------------------------------------------ multi-hop queries
    @staticmethod
    def t_norm(a: torch.Tensor, b: torch.Tensor, tnorm: str = "min") -> torch.Tensor:
        return torch.min(a, b) if "min" in tnorm else a * b

    @staticmethod
    def tensor_t_norm(subquery_scores: torch.Tensor, tnorm: str = "min"):
        if tnorm == "min":
            return torch.min(subquery_scores, dim=0)
        raise NotImplementedError(f"{tnorm} is not implemented")

    @staticmethod
    def t_conorm(a: torch.Tensor, b: torch.Tensor, tconorm: str = "min") -> torch.Tensor:
        return torch.max(a, b) if "min" in tconorm else (a + b) - (a * b)

    @staticmethod
    def negnorm(x: torch.Tensor, lambda_: float, neg_norm: str = "standard") -> torch.Tensor:
        if "standard" in neg_norm:
            return 1 - x
        if "sugeno" in neg_norm:
            return (1 - x) / (1 + lambda_ * x)
        if "yager" in neg_norm:
            return (1 - torch.pow(x, lambda_)) ** (1 / lambda_)
        raise ValueError(neg_norm)

    @torch.no_grad()
    def _atom(self, head_ids: torch.Tensor, rel: str) -> torch.Tensor:
        """Logits ``[len(head_ids), |E|]`` of ``(head, rel, ?)`` in one model call."""
        dev = self.model.device
        x = torch.stack((head_ids.to(dev), torch.full_like(head_ids, self.relation_to_idx[rel]).to(dev)), dim=1)
        return self.model(x).view(head_ids.numel(), -1).cpu()

    def _project(self, scores: torch.Tensor, rel: str, k: int, tnorm: str, negate=None) -> torch.Tensor:
        """Relational projection of a score vector: keep the ``k`` best intermediate entities, score their
        tails in one batch and take ``max_beam tnorm(beam score, atom score)``."""
        top, idx = torch.topk(scores, k)
        atom = self._atom(idx, rel)
        if negate is not None:
            atom = negate(atom)
        return torch.max(self.t_norm(top.view(-1, 1).expand_as(atom), atom, tnorm), dim=0)[0]

    def _chain(self, anchor: str, rels: Tuple[str, ...], k: int, tnorm: str, neg) -> torch.Tensor:
        """Scores of a path query ``anchor -r1-> … -rn-> ?``; a trailing ``'n'`` negates the last atom."""
        rels = tuple(rels)
        negate_last = len(rels) > 1 and rels[-1] == "n"
        if negate_last:
            rels = rels[:-1]
        s = self._atom(self._ent_ids(anchor), rels[0]).squeeze(0)
        if negate_last and len(rels) == 1:
            return neg(s)
        for i, r in enumerate(rels[1:], start=1):
            last = i == len(rels) - 1
            s = self._project(s, r, k, tnorm, negate=neg if (negate_last and last) else None)
        return s

    def return_multi_hop_query_results(self, scores, k: int, only_scores: bool):
        if only_scores:
            return scores
        return sorted(zip(self.entity_to_idx.keys(), scores), key=lambda x: x[1], reverse=True)[:k]

    def single_hop_query_answering(self, query: tuple, only_scores: bool = True, k: int = None):
        h, r = query
        s = self._atom(self._ent_ids(h), r[0]).squeeze(0)
        return self.return_multi_hop_query_results(s, k, only_scores)

    def answer_multi_hop_query(self, query_type: str = None, query=None, queries=None, tnorm: str = "prod",
                               neg_norm: str = "standard", lambda_: float = 0.0, k: int = 10, only_scores=False):
        """Answer an EPFO(+negation) query of type 1p 2p 3p 2i 3i ip pi 2in 3in inp pin pni 2u up by
        continuous query decomposition: atoms are model logits, conjunction a t-norm, disjunction a t-conorm,
        projection a beam of width ``k`` (reference ``knowledge_graph_embeddings.py:670-1170``)."""
        if queries is not None:
            assert query is None
            return [self.answer_multi_hop_query(query_type=query_type, query=q, tnorm=tnorm, neg_norm=neg_norm,
                                                lambda_=lambda_, k=k, only_scores=only_scores) for q in queries]
        assert len(self.entity_to_idx) >= k >= 0
        if query_type not in QUERY_NAME.values():
            raise ValueError(f"Invalid query type: {query_type}")
        neg = lambda x: self.negnorm(x, lambda_, neg_norm)  # noqa: E731
        chain = lambda e, rs: self._chain(e, rs if isinstance(rs, tuple) else (rs,), k, tnorm, neg)  # noqa: E731
        if query_type in ("1p", "2p", "3p"):
            e, rs = query
            s = chain(e, tuple(rs))
            return self.return_multi_hop_query_results(s, k, only_scores)
        if query_type in ("2i", "3i", "2in", "3in", "pi", "pin", "pni"):
            parts = [chain(e, tuple(rs)) for e, rs in query]
            s = parts[0]
            for p in parts[1:]:
                s = self.t_norm(s, p, tnorm)
        elif query_type == "2u":
            (e1, r1), (e2, r2) = query[0], query[1]
            s = self.t_conorm(chain(e1, tuple(r1)), chain(e2, tuple(r2)), tnorm)
        elif query_type in ("ip", "inp", "up"):
            inner, (r_last,) = query[0], query[1]
            (e1, r1), (e2, r2) = inner[0], inner[1]
            a, b = chain(e1, tuple(r1)), chain(e2, tuple(r2))
            mid = self.t_conorm(a, b, tnorm) if query_type == "up" else self.t_norm(a, b, tnorm)
            s = self._project(mid, r_last, k, tnorm)
        else:
            raise RuntimeError(f"Incorrect query_structure {query_type}")
        if only_scores:
            return s
        return sorted(zip(self.entity_to_idx.keys(), s), key=lambda x: x[1], reverse=True)

    def find_missing_triples(self, confidence: float, entities: List[str] = None, relations: List[str] = None,
                             topk: int = 10, at_most: int = sys.maxsize) -> Set:
        """``(h, r, t)`` predicted with probability ≥ ``confidence`` that are not in the training split."""
        assert 1.0 >= confidence >= 0.0 and topk >= 1
        ents = list(self.entity_to_idx) if entities is None else entities
        rels = list(self.relation_to_idx) if relations is None else relations
        known = set(map(tuple, np.asarray(self.train_set).tolist()))
        out: Set = set()
        for r in rels:
            res = self.predict_topk(h=ents, r=[r], topk=topk)
            for h, row in zip(ents, res):
                for t, p in row:
                    if p < confidence:
                        break
                    if (self.entity_to_idx[h], self.relation_to_idx[r], self.entity_to_idx[t]) in known:
                        continue
                    out.add((h, r, t))
                    if len(out) == at_most:
                        return out
        return out

    # ------------------------------------------------------------------ fine-tuning
    def train_triples(self, h: List[str], r: List[str], t: List[str], labels: List[float], iteration: int = 2,
                      optimizer=None):
        assert len(h) == len(r) == len(t) == len(labels)
        x, y = self.construct_input_and_output(h, r, t, labels)
        x, y = x.to(self.model.device), y.to(self.model.device)
        self.set_model_train_mode()
        optimizer = optimizer or torch.optim.Adam(self.model.parameters(), lr=0.1)
        for it in range(iteration):
            optimizer.zero_grad()
            out = self.model(x)
            loss = self.model.loss(out, y)
            print(f"Iteration:{it}\t Loss:{loss.item()}\t Outputs:{out.detach().mean()}")
            loss.backward()
            optimizer.step()
        self.set_model_eval_mode()
        with torch.no_grad():
            print(f"Eval Mode:\tLoss:{self.model.loss(self.model(x), y).item()}")

    def train_k_vs_all(self, h, r, iteration: int = 1, lr: float = 0.001):
        """Fit ``(h, r, ·)`` against the multi-hot vector of the tails known in the stored training split."""
        assert len(h) == 1
        hi, ri = self.entity_to_idx[h[0]], self.relation_to_idx[r[0]]
        ts = np.asarray(self.train_set)
        tails = ts[(ts[:, 0] == hi) & (ts[:, 1] == ri)][:, 2]
        if tails.size == 0:
            return
        x = torch.LongTensor([[hi, ri]]).to(self.model.device)
        y = torch.zeros(1, self.num_entities, device=self.model.device)
        y[0, torch.as_tensor(tails).long()] = 1.0
        self.set_model_train_mode()
        opt = torch.optim.Adam(self.model.parameters(), lr=lr, weight_decay=0.00001)
        for it in range(iteration):
            opt.zero_grad()
            loss = self.model.loss(self.model(x), y)
            loss.backward()
            opt.step()
        self.set_model_eval_mode()

    def train(self, kg, lr: float = 0.1, epoch: int = 10, batch_size: int = 32, neg_sample_ratio: int = 10,
              num_workers: int = 1) -> None:
        """Continue training on ``kg.train_set`` with negative sampling and Adam."""
        ds = TriplePredictionDataset(kg.train_set, len(kg.entity_to_idx), len(kg.relation_to_idx), neg_sample_ratio)
        ds.to(self.model.device)
        loader = BatchLoader(ds, batch_size=batch_size, shuffle=True)
        n = len(ds)

        def avg_loss():
            tot = 0.0
            with torch.no_grad():
                for x, y in loader:
                    tot += float(self.model.loss(self.model(x), y))
            return tot / n

        self.set_model_eval_mode()
        first = avg_loss()
        self.set_model_train_mode()
        opt = torch.optim.Adam(self.model.parameters(), lr=lr)
        for ep in range(epoch):
            tot = 0.0
            for x, y in loader:
                opt.zero_grad()
                loss = self.model.loss(self.model(x), y)
                tot += float(loss.detach())
                loss.backward()
                opt.step()
            print(f"Epoch={ep}\t Avg. Loss per epoch: {tot / n:.3f}")
        self.set_model_eval_mode()
        print(f"On average Improvement: {first - avg_loss():.3f}")

    # ------------------------------------------------------------------ literals
    def _maybe_load_literal_model(self) -> None:
        lm = os.path.join(self.path, "literal_model.pt")
        at = os.path.join(self.path, "attribute_to_idx.csv")
        if not (os.path.isfile(lm) and os.path.isfile(at)) or not hasattr(self.model, "entity_embeddings"):
            return
        df = pd.read_csv(at, index_col=0)
        self.data_property_to_idx = {a: int(i) for i, a in zip(df.index, df["attribute"])}
        self.idx_to_data_property = {v: k for k, v in self.data_property_to_idx.items()}
        sd = torch.load(lm, map_location="cpu", weights_only=False)
        model = LiteralEmbeddings(len(self.data_property_to_idx), self.model.embedding_dim,
                                  self.model.entity_embeddings,
                                  gate_residual=any(k.startswith("gated_residual_proj") for k in sd))
        model.load_state_dict(sd)
        model.eval()
        self.literal_model = model
        norm = os.path.join(self.path, "literal_normalization.json")
        if os.path.isfile(norm):
            self.literal_dataset = _NormOnly(load_json(norm))

    def train_literals(self, train_file_path: str = None, num_epochs: int = 100, lit_lr: float = 0.001,
                       lit_normalization_type: str = "z-norm", batch_size: int = 1024, sampling_ratio: float = None,
                       random_seed=1, loader_backend: str = "pandas", freeze_entity_embeddings: bool = True,
                       gate_residual: bool = True, device: str = None, suffle_data: bool = True):
        """Train the literal regressor (L1 loss, Adam) on ``(entity, attribute, value)`` rows of a file; stores
        ``literal_model.pt`` and ``attribute_to_idx.csv`` in the run directory
        (reference ``dicee/abstracts.py:769-871``)."""
        torch.manual_seed(random_seed)
        dev = torch.device(device) if device else self.model.device
        ds = LiteralDataset(train_file_path, self.entity_to_idx, lit_normalization_type, sampling_ratio,
                            loader_backend)
        self.data_property_to_idx = ds.data_property_to_idx
        lit = LiteralEmbeddings(ds.num_data_properties, self.model.embedding_dim, self.model.entity_embeddings,
                                freeze_entity_embeddings=freeze_entity_embeddings, gate_residual=gate_residual).to(dev)
        opt = torch.optim.Adam(lit.parameters(), lr=lit_lr)
        ds.to(dev)
        loader = BatchLoader(ds, batch_size=batch_size, shuffle=suffle_data, seed=random_seed)
        lit.train()
        loss_log = {"lit_loss": []}
        for _ in range(num_epochs):
            tot, nb = 0.0, 0
            for bx, by in loader:
                opt.zero_grad()
                loss = F.l1_loss(lit(bx[:, 0], bx[:, 1]), by)
                loss.backward()
                opt.step()
                tot += float(loss.detach())
                nb += 1
            loss_log["lit_loss"].append(tot / max(nb, 1))
        lit.eval()
        self.literal_model, self.literal_dataset = lit, ds
        torch.save({k: v.cpu() for k, v in lit.state_dict().items()}, os.path.join(self.path, "literal_model.pt"))
        self.idx_to_data_property = {v: k for k, v in self.data_property_to_idx.items()}
        pd.DataFrame.from_dict(self.idx_to_data_property, orient="index", columns=["attribute"]).to_csv(
            os.path.join(self.path, "attribute_to_idx.csv"))
        from .io.checkpoint import write_json
        write_json(ds.normalization_params, os.path.join(self.path, "literal_normalization.json"))
        return loss_log

    @torch.no_grad()
    def predict_literals(self, entity: StrOrList = None, attribute: StrOrList = None,
                         denormalize_preds: bool = True) -> np.ndarray:
        if self.literal_model is None:
            raise RuntimeError("Literal model is not trained or loaded.")
        if entity is None or attribute is None:
            raise RuntimeError("Entity and Attribute cannot be of type None")
        entity = [entity] if isinstance(entity, str) else entity
        attribute = [attribute] if isinstance(attribute, str) else attribute
        assert len(entity) == len(attribute), "Entity and attribute lists must be of equal length"
        dev = self.literal_model.device
        e = torch.LongTensor([self.entity_to_idx[i] for i in entity]).to(dev)
        a = torch.LongTensor([self.data_property_to_idx[i] for i in attribute]).to(dev)
        preds = self.literal_model(e, a).cpu().numpy()
        if denormalize_preds and self.literal_dataset is not None:
            preds = LiteralDataset.denormalize(preds, attribute, self.literal_dataset.normalization_params)
        return preds

    # ------------------------------------------------------------------ generation (BytE)
    def generate(self, h: str = "", r: str = "", max_new_tokens: Optional[int] = None) -> str:
        """Greedy continuation of ``"h r "`` by a BytE language model, decoded back to text."""
        assert self.configs.get("byte_pair_encoding")
        space = self.enc.encode(" ")[0]
        ids = [*self.enc.encode(h), space, *self.enc.encode(r), space]
        bs = self.model.config.block_size
        x = torch.LongTensor([ids[-bs:]]).to(self.model.device)
        out = self.model.generate(x, max_new_tokens or bs, temperature=self.model.temperature, top_k=1)
        return self.enc.decode(out[0, x.shape[1]:].tolist())


class _NormOnly:
    """Carrier of literal normalisation constants reloaded from disk."""

    def __init__(self, params: Dict):
        self.normalization_params = params

    @staticmethod
    def load_and_validate_literal_data(file_path: str, loader_backend: str = "pandas"):
        return LiteralDataset.load_and_validate_literal_data(file_path, loader_backend)
