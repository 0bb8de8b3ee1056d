"""Stand-alone link-prediction evaluation functions.

Same names and return values (``{'H@1','H@3','H@10','MRR'}``) as the reference module
``dicee/evaluation/link_prediction.py``; all of them are batched through
:mod:`.ranking` instead of looping over triples in Python.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .ranking import (filter_coordinates, filtered_rank_from_scores, head_and_tail_ranks, metrics_from_ranks,
                      tail_ranks)


def _index_string_triples(model, triples) -> np.ndarray:
    e2i, r2i = model.entity_to_idx, model.relation_to_idx
    return np.array([(e2i[h], r2i[r], e2i[t]) for h, r, t in triples], dtype=np.int64)


def evaluate_lp(model, triple_idx, num_entities: int, er_vocab, re_vocab, info: str = "Eval Starts",
                batch_size: int = 128, chunk_size: int = 1000) -> Dict[str, float]:
    """Head **and** tail filtered ranking through the triple-scoring path; metrics are divided by ``2N``
    (reference ``link_prediction.py:352-473``).  With ``er_vocab`` / ``re_vocab`` ``None`` the ranking is raw."""
    model.eval()
    hr, tr = head_and_tail_ranks(model, triple_idx, num_entities, er_vocab, re_vocab, batch_size, chunk_size)
    return metrics_from_ranks(torch.cat((hr, tr)), divisor=2 * len(triple_idx))


def evaluate_link_prediction_performance(model, triples, er_vocab, re_vocab) -> Dict[str, float]:
    """``model`` is a :class:`KGE` wrapper, ``triples`` a list of string triples; predicts missing heads and
    missing tails (reference ``link_prediction.py:23-114``)."""
    idx = _index_string_triples(model, triples)
    return evaluate_lp(model.model, idx, model.num_entities, er_vocab, re_vocab)


def evaluate_link_prediction_performance_with_reciprocals(model, triples, er_vocab) -> Dict[str, float]:
    """Tail-only filtered ranking for models trained with reciprocal triples
    (reference ``link_prediction.py:117-174``)."""
    idx = _index_string_triples(model, triples)
    model.model.eval()
    ranks = tail_ranks(model.model, idx, er_vocab, batch_size=1024)
    return metrics_from_ranks(ranks, divisor=len(idx))


def _bpe_rows(model, items: List[str]) -> torch.Tensor:
    return torch.LongTensor([model.get_bpe_token_representation(i) for i in items])


@torch.no_grad()
def evaluate_link_prediction_performance_with_bpe_reciprocals(model, within_entities: List[str],
                                                              triples: List[List[str]], er_vocab) -> Dict[str, float]:
    """Tail ranking for byte-pair-encoded triple scorers: every entity of ``within_entities`` is scored as
    tail (reference ``link_prediction.py:177-237``)."""
    model.model.eval()
    ent_tok = _bpe_rows(model, within_entities)
    pos = {e: i for i, e in enumerate(within_entities)}
    ranks = []
    for h, r, t in triples:
        ht, rt = _bpe_rows(model, [h]), _bpe_rows(model, [r])
        n = len(within_entities)
        x = torch.stack((ht.expand(n, -1), rt.expand(n, -1), ent_tok), dim=1)
        s = model.model(x).reshape(1, -1)
        filt = [pos[e] for e in er_vocab.get((h, r), []) if e in pos]
        fr = torch.zeros(len(filt), dtype=torch.long)
        ranks.append(filtered_rank_from_scores(s, torch.tensor([pos[t]]), fr, torch.tensor(filt, dtype=torch.long)))
    return metrics_from_ranks(torch.cat(ranks), divisor=len(triples))


@torch.no_grad()
def evaluate_link_prediction_performance_with_bpe(model, within_entities: List[str], triples: List[Tuple[str]],
                                                  er_vocab, re_vocab) -> Dict[str, float]:
    """Head and tail ranking for byte-pair-encoded triple scorers (reference ``link_prediction.py:240-349``)."""
    model.model.eval()
    ent_tok = _bpe_rows(model, within_entities)
    pos = {e: i for i, e in enumerate(within_entities)}
    n = len(within_entities)
    ranks = []
    for h, r, t in triples:
        ht, rt, tt = _bpe_rows(model, [h]), _bpe_rows(model, [r]), _bpe_rows(model, [t])
        s_tail = model.model(torch.stack((ht.expand(n, -1), rt.expand(n, -1), ent_tok), dim=1)).reshape(1, -1)
        s_head = model.model(torch.stack((ent_tok, rt.expand(n, -1), tt.expand(n, -1)), dim=1)).reshape(1, -1)
        ft = [pos[e] for e in er_vocab.get((h, r), []) if e in pos]
        fh = [pos[e] for e in re_vocab.get((r, t), []) if e in pos]
        ranks.append(filtered_rank_from_scores(s_tail, torch.tensor([pos[t]]), torch.zeros(len(ft), dtype=torch.long),
                                               torch.tensor(ft, dtype=torch.long)))
        ranks.append(filtered_rank_from_scores(s_head, torch.tensor([pos[h]]), torch.zeros(len(fh), dtype=torch.long),
                                               torch.tensor(fh, dtype=torch.long)))
    return metrics_from_ranks(torch.cat(ranks), divisor=2 * len(triples))


@torch.no_grad()
def evaluate_bpe_lp(model, triple_idx: List[Tuple], all_bpe_shaped_entities, er_vocab, re_vocab,
                    info: str = "Eval Starts") -> Dict[str, float]:
    """Head and tail ranking on padded token triples against ``all_bpe_shaped_entities`` (list of
    ``(string, tokens, padded tokens)``); vocabularies are keyed by padded-token tuples
    (reference ``link_prediction.py:477-579``)."""
    model.eval()
    ent = torch.tensor([s for (_, _, s) in all_bpe_shaped_entities], dtype=torch.long)
    pos = {tuple(s): i for i, (_, _, s) in enumerate(all_bpe_shaped_entities)}
    n = ent.shape[0]
    ranks = []
    for h, r, t in triple_idx:
        h, r, t = tuple(h), tuple(r), tuple(t)
        ht, rt, tt = (torch.tensor([v], dtype=torch.long) for v in (h, r, t))
        s_tail = model(torch.stack((ht.expand(n, -1), rt.expand(n, -1), ent), dim=1)).reshape(1, -1)
        s_head = model(torch.stack((ent, rt.expand(n, -1), tt.expand(n, -1)), dim=1)).reshape(1, -1)
        ft = [pos[tuple(e)] for e in (er_vocab or {}).get((h, r), []) if tuple(e) in pos]
        fh = [pos[tuple(e)] for e in (re_vocab or {}).get((r, t), []) if tuple(e) in pos]
        ranks.append(filtered_rank_from_scores(s_tail, torch.tensor([pos[t]]), torch.zeros(len(ft), dtype=torch.long),
                                               torch.tensor(ft, dtype=torch.long)))
        ranks.append(filtered_rank_from_scores(s_head, torch.tensor([pos[h]]), torch.zeros(len(fh), dtype=torch.long),
                                               torch.tensor(fh, dtype=torch.long)))
    return metrics_from_ranks(torch.cat(ranks), divisor=2 * len(triple_idx))


@torch.no_grad()
def evaluate_lp_bpe_k_vs_all(model, triples: List[List[str]], er_vocab=None, batch_size: Optional[int] = None,
                             func_triple_to_bpe_representation=None, str_to_bpe_entity_to_idx=None) -> Dict[str, float]:
    """Tail ranking of string triples with a byte-pair-encoded all-entity scorer
    (reference ``link_prediction.py:582-642``)."""
    model.eval()
    bs = batch_size or 128
    ranks = []
    for i in range(0, len(triples), bs):
        chunk = triples[i:i + bs]
        tok = torch.LongTensor([func_triple_to_bpe_representation(list(tr)) for tr in chunk])
        scores = model(tok[:, :2, :])
        tgt = torch.tensor([str_to_bpe_entity_to_idx[t] for _, _, t in chunk])
        rows, cols = [], []
        for j, (h, r, _) in enumerate(chunk):
            for e in (er_vocab or {}).get((h, r), []):
                if e in str_to_bpe_entity_to_idx:
                    rows.append(j)
                    cols.append(str_to_bpe_entity_to_idx[e])
        ranks.append(filtered_rank_from_scores(scores, tgt, torch.tensor(rows, dtype=torch.long),
                                               torch.tensor(cols, dtype=torch.long)))
    return metrics_from_ranks(torch.cat(ranks), divisor=len(triples))
