"""Vectorised filtered ranking.

The reference computes filtered ranks with a Python loop per row (assign ``-inf`` to the filter indices,
full ``torch.sort``, ``torch.where`` per row; ``dicee/evaluation/evaluator.py:484-508``).  The rank of the
target only depends on *how many* candidates beat it, so here

    ``rank = 1 + #{j : s_j > s_target} − #{j ∈ known answers, j ≠ target : s_j > s_target}``

is evaluated with two reductions per batch and a sparse gather driven by the CSR filter vocabulary, with no
sort and no per-row Python.  Ties are resolved optimistically (only strictly larger scores count), which is
what a stable descending sort gives when the target is met first.  The same decomposition is what the fused
GEMM+rank CUDA kernel implements for sharded tables.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..data.vocab import PairCSR

ALL_HITS_RANGE = list(range(1, 11))


def metrics_from_ranks(ranks: torch.Tensor, divisor: Optional[float] = None,
                       hits: Sequence[int] = (1, 3, 10)) -> Dict[str, float]:
    """H@k and MRR from a tensor of ranks; ``divisor`` defaults to the number of ranks
    (reference ``dicee/evaluation/utils.py:41-98``)."""
    ranks = ranks.double()
    n = float(divisor if divisor is not None else max(ranks.numel(), 1))
    out = {f"H@{k}": float((ranks <= k).sum()) / n for k in hits}
    out["MRR"] = float((1.0 / ranks).sum()) / n
    return out


def filtered_rank_from_scores(scores: torch.Tensor, target: torch.Tensor,
                              filt_rows: Optional[torch.Tensor] = None,
                              filt_cols: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Ranks ``[B]`` of ``target [B]`` inside ``scores [B, N]`` ignoring the (row, col) filter entries."""
    B = scores.shape[0]
    ar = torch.arange(B, device=scores.device)
    tgt = scores[ar, target]
    greater = (scores > tgt.unsqueeze(1)).sum(dim=1)
    if filt_rows is not None and filt_rows.numel():
        beat = (scores[filt_rows, filt_cols] > tgt[filt_rows]) & (filt_cols != target[filt_rows])
        greater = greater - torch.zeros_like(greater).index_add_(0, filt_rows, beat.to(greater.dtype))
    return greater + 1


def _dict_filter(vocab: Dict, keys: Iterable[Tuple[int, int]], device) -> Tuple[torch.Tensor, torch.Tensor]:
    rows: List[int] = []
    cols: List[int] = []
    for i, k in enumerate(keys):
        v = vocab.get(k, ()) if hasattr(vocab, "get") else vocab[k]
        rows.extend([i] * len(v))
        cols.extend(v)
    return (torch.tensor(rows, dtype=torch.long, device=device), torch.tensor(cols, dtype=torch.long, device=device))


def filter_coordinates(vocab, a: torch.Tensor, b: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(row, col) pairs of all known answers for the query pairs ``(a_i, b_i)``; ``vocab`` is a
    :class:`PairCSR` or a dict ``(a, b) -> list``."""
    if vocab is None:
        e = torch.zeros(0, dtype=torch.long, device=a.device)
        return e, e
    if isinstance(vocab, PairCSR):
        return vocab.batch_rows_cols(a, b)
    return _dict_filter(vocab, zip(a.tolist(), b.tolist()), a.device)


def filter_csr(vocab, a: torch.Tensor, b: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-query CSR ``(ptr [B+1] int64, cols int32)`` of the known answers of the pairs ``(a_i, b_i)``."""
    rows, cols = filter_coordinates(vocab, a, b)
    ptr = torch.zeros(a.shape[0] + 1, dtype=torch.int64, device=a.device)
    if rows.numel():
        ptr[1:] = torch.cumsum(torch.bincount(rows, minlength=a.shape[0]), 0)
    return ptr, cols.to(torch.int32)


def _use_fused(model, fused: Optional[bool]) -> bool:
    if fused is False:
        return False
    from ..ops import eval_rank
    ok = eval_rank.supports(model)
    if fused and not ok:
        raise RuntimeError("fused ranking requested but the model is not bilinear / not on a CUDA device / too wide")
    return ok


@torch.no_grad()
def fused_tail_ranks(model, triples: torch.Tensor, er_vocab, batch_size: int = 4096, ranker=None) -> torch.Tensor:
    """:func:`tail_ranks` through the tcgen05 ranking kernel: no ``[B, |E|]`` score matrix, no sort.  The tensor
    cores score bf16-rounded operands; entities whose score falls within the rounding margin of the target are
    re-scored in fp32, so the ranks are those of an fp32 evaluation.  Should the list of such entities overflow
    (targets ranked in the middle of a very large table), the batch is ranked from the bf16 scores alone."""
    from ..ops import eval_rank
    from ..ops.kernels import KernelError
    ranker = ranker or eval_rank.ranker_for_model(model)
    dev = ranker.device
    out = []
    for i in range(0, triples.shape[0], batch_size):
        b = triples[i:i + batch_size].to(dev)
        q, _ = eval_rank.model_queries(model, b[:, :2])
        ptr, cols = filter_csr(er_vocab, b[:, 0], b[:, 1])
        try:
            r = ranker.ranks(q, b[:, 2], ptr, cols).cpu()
            ranker.check()          # the ranks are on the host already: reading the status words costs nothing more
        except KernelError:
            if not ranker.exact:
                raise
            ranker.exact = False
            try:
                r = ranker.ranks(q, b[:, 2], ptr, cols).cpu()
                ranker.check()
            finally:
                ranker.exact = True
        out.append(r)
    return torch.cat(out) if out else torch.zeros(0, dtype=torch.long)


@torch.no_grad()
def tail_ranks(model, triples: torch.Tensor, er_vocab, batch_size: int = 1024, device=None,
               fused: Optional[bool] = None) -> torch.Tensor:
    """Filtered rank of the true tail among all entities for every ``(h, r, t)`` row.  ``fused``: ``None`` picks
    the tcgen05 ranking kernel whenever the model supports it, ``False`` forces the PyTorch path."""
    device = device or getattr(model, "device", torch.device("cpu"))
    out = []
    triples = torch.as_tensor(np.asarray(triples)).long()
    if _use_fused(model, fused):
        return fused_tail_ranks(model, triples, er_vocab, max(batch_size, 1024))
    for i in range(0, triples.shape[0], batch_size):
        b = triples[i:i + batch_size].to(device)
        scores = model(b[:, :2])
        fr, fc = filter_coordinates(er_vocab, b[:, 0], b[:, 1])
        out.append(filtered_rank_from_scores(scores, b[:, 2], fr, fc).cpu())
    return torch.cat(out) if out else torch.zeros(0, dtype=torch.long)


@torch.no_grad()
def relation_ranks(model, triples: torch.Tensor, ee_vocab, batch_size: int = 1024, device=None) -> torch.Tensor:
    """Filtered rank of the true relation for every row (relation-prediction models)."""
    device = device or getattr(model, "device", torch.device("cpu"))
    out = []
    triples = torch.as_tensor(np.asarray(triples)).long()
    for i in range(0, triples.shape[0], batch_size):
        b = triples[i:i + batch_size].to(device)
        scores = model.forward_k_vs_all(x=b[:, [0, 2]])
        fr, fc = filter_coordinates(ee_vocab, b[:, 0], b[:, 2])
        out.append(filtered_rank_from_scores(scores, b[:, 1], fr, fc).cpu())
    return torch.cat(out) if out else torch.zeros(0, dtype=torch.long)


@torch.no_grad()
def _all_entity_triple_scores(model, fixed_a: torch.Tensor, rel: torch.Tensor, slot: str, num_entities: int,
                              chunk_size: int) -> torch.Tensor:
    """Scores ``[B, |E|]`` of every entity placed in ``slot`` ('head' or 'tail') through ``forward_triples``."""
    B = fixed_a.shape[0]
    dev = fixed_a.device
    out = torch.empty(B, num_entities, device=dev)
    for s in range(0, num_entities, chunk_size):
        e = torch.arange(s, min(s + chunk_size, num_entities), device=dev)
        C = e.numel()
        cand = e.repeat(B)
        a = fixed_a.repeat_interleave(C)
        r = rel.repeat_interleave(C)
        x = torch.stack((cand, r, a), dim=1) if slot == "head" else torch.stack((a, r, cand), dim=1)
        out[:, s:s + C] = model(x).reshape(B, C)
    return out


@torch.no_grad()
def head_and_tail_ranks(model, triples, num_entities: int, er_vocab, re_vocab, batch_size: int = 128,
                        chunk_size: int = 1000, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Filtered ranks of the true head and of the true tail for every triple, scoring all entities
    through the triple path (the protocol of models trained without reciprocal triples; reference
    ``dicee/evaluation/link_prediction.py:352-473``)."""
    device = device or getattr(model, "device", torch.device("cpu"))
    triples = torch.as_tensor(np.asarray(triples)).long()
    hr, tr = [], []
    for i in range(0, triples.shape[0], batch_size):
        b = triples[i:i + batch_size].to(device)
        h, r, t = b[:, 0], b[:, 1], b[:, 2]
        s_tail = _all_entity_triple_scores(model, h, r, "tail", num_entities, chunk_size)
        fr, fc = filter_coordinates(er_vocab, h, r)
        tr.append(filtered_rank_from_scores(s_tail, t, fr, fc).cpu())
        s_head = _all_entity_triple_scores(model, t, r, "head", num_entities, chunk_size)
        fr, fc = filter_coordinates(re_vocab, r, t)
        hr.append(filtered_rank_from_scores(s_head, h, fr, fc).cpu())
    z = torch.zeros(0, dtype=torch.long)
    return (torch.cat(hr) if hr else z), (torch.cat(tr) if tr else z)
